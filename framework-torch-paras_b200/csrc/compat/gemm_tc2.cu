// The projection GEMM on CTA pairs: C[M, N] = A[M, K] * B[N, K]^T (either operand also transposed, batched) with 256 x 256 output tiles, each
// computed by two CTAs of a cluster (`tcgen05.mma.cta_group::2`, M = 256).  The call sites are the same as
// gemm_tc.cu's: aten::linear / addmm / mm of the reference (csrc/ops/vision_ops.cpp:248-309, 388-423) and
// the gate/up projection with SwiGLU (csrc/ops/rms_swiglu_ops.cpp:77-104).
//
// Why pairs.  The single-CTA kernel (gemm_tc.cu) moves 48 KB of operands into shared memory per K step
// of a 128 x 256 tile and is bound by the bytes it keeps in flight (three stages ahead; one stage less
// costs it 9-14 %).  In a pair each CTA holds its own 128 rows of A and HALF of the B tile (128 of the
// 256 weight rows); the MMA reads both halves, so a CTA needs 32 KB per K step for the same FLOPs and
// the same shared memory holds six stages instead of four.
//
// Roles per CTA (192 threads): warps 0-3 epilogue (TMEM -> registers -> swizzled shared memory -> TMA
// store of the CTA's own 128 rows), warp 4 allocates TMEM and, in the pair's first CTA only, issues every
// MMA, warp 5 is the TMA producer of the CTA's own operand halves.  Barriers: a stage's `full` barrier
// lives in the first CTA and counts the bytes of both CTAs' loads (the second CTA's TMA signals it across
// the cluster); `empty` and `accumulator full` exist in both CTAs and the issuing thread commits to each
// of them (its own, and the peer's through a mapped address); `accumulator empty` lives in the first CTA
// and takes the arrivals of both CTAs' epilogue warps.  Every wait is bounded (tc::mbar_wait).
//
// SwiGLU epilogue: the first CTA loads 128 gate-weight rows and the second 128 up-weight rows, so the
// N = 256 MMA leaves [gate | up] side by side in each CTA's accumulator exactly as in gemm_tc.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "tc_prims.cuh"
#include "tma_host.cuh"
#include "gemm_internal.cuh"

namespace pb {
namespace {

using namespace tc;

constexpr int BMC = 128;                     // rows of a tile per CTA (the pair's tile has 256)
constexpr int BN = 256, BK = 64;
constexpr int kABytes = BMC * BK * 2;        // 16 KB
constexpr int kBBytes = (BN / 2) * BK * 2;   // 16 KB: this CTA's half of the B tile
constexpr int kStepBytes = kABytes + kBBytes;
// Two K steps share a stage and its barriers: the issuing thread then pays one wait and two commits per
// eight MMAs instead of per four (a wait costs it 250-350 cycles even on a barrier that completed long ago,
// against 524 cycles of tensor-pipe work in four MMAs).
constexpr int kStepsPerStage = 2;
constexpr int kStages = 3;
constexpr int kStageBytes = kStepsPerStage * kStepBytes;
constexpr int kEpiWarps = 4, kMmaWarp = 4, kLoadWarp = 5, kThreads = 192;
constexpr int kTmemCols = 512;               // two accumulators of 256 columns
constexpr int kOutStage = 32 * 128;
constexpr int kGroupM = 8;                   // tile order: 8 row blocks (of 256 rows) at a time
constexpr int kSmemOut = kStages * kStageBytes;
constexpr int kSmemBars = kSmemOut + kEpiWarps * 2 * kOutStage;
constexpr int kBarFull = 0, kBarEmpty = kStages, kBarAccFull = 2 * kStages, kBarAccEmpty = 2 * kStages + 2;
constexpr int kNumBars = 2 * kStages + 4;
constexpr int kSmemMisc = kSmemBars + kNumBars * 8;
constexpr int kSmemTotal = kSmemMisc + 16;
static_assert(kSmemTotal <= 232448, "shared memory of a CTA");

enum { kEpiNone = 0, kEpiBias = 1, kEpiSwiglu = 2, kEpiRowScale = 5 };

struct Params {
    int M, N, K;
    int batch;
    int tiles_m, tiles_n, tiles;   // per batch: tiles of 256 rows x (256 | 128 with SwiGLU) columns; tiles = all batches
    int k_iters;
    const void* bias;
    const float* row_scale;
    int* status;
};

struct Tile { int b, m0, n0; };

__device__ __forceinline__ Tile get_tile(const Params& p, int id, int n_per_tile) {
    const int per_batch = p.tiles_m * p.tiles_n;
    Tile t;
    t.b = id / per_batch;
    id -= t.b * per_batch;
    const int in_group = kGroupM * p.tiles_n;
    const int group = id / in_group;
    const int first_m = group * kGroupM;
    const int gm = min(p.tiles_m - first_m, kGroupM);
    const int q = id - group * in_group;
    t.m0 = (first_m + q % gm) * (2 * BMC);
    t.n0 = (q / gm) * n_per_tile;
    return t;
}

// ---- the cluster-level forms of the primitives ------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// the address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' 128 rows] * B[both CTAs' halves]
__device__ __forceinline__ void mma2_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival at the barrier (a shared::cluster address: this CTA's or the peer's) once every MMA this
// thread issued so far has completed in both CTAs.
__device__ __forceinline__ void tc_commit2(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load into this CTA's shared memory whose bytes count on a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma2_load_3d(uint32_t dst_smem, const CUtensorMap* map, uint32_t cluster_bar,
                                             int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// A_KM: A is given as [K, M] rows (the transposed operand of a weight gradient); B_KN: B as [K, N] rows
// (mm / bmm, and the input gradient of a linear layer).  Such an operand lands in shared memory as
// 64-column slabs of 64 K-rows and is read through MN-major descriptors, as in gemm_tc.cu.
template <bool BF16, bool A_KM, bool B_KN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c,
                const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    auto bar = [&](int i) { return smem_base + kSmemBars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + kSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + kSmemMisc + 4);
    constexpr int kNPerTile = EPI == kEpiSwiglu ? BN / 2 : BN;   // output columns per tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = int(blockIdx.x >> 1), pairs = int(gridDim.x >> 1);
    // (every CTA of the grid takes the same branch: the base of dynamic shared memory is the same in all)
    if (smem_base & 1023u) {
        if (threadIdx.x == 0) {
            *p.status = int(0x40000000u | (1u << 29));
            __threadfence_system();
        }
        return;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i)
            mbar_init(bar(i), i >= kBarAccEmpty ? uint32_t(2 * kEpiWarps) : 1u);
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc2(smem_base + kSmemMisc, kTmemCols);
        tmem_relinquish2();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (EPI == kEpiSwiglu) tma_prefetch_desc(&map_b2);
        tma_prefetch_desc(&map_c);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised before anything arrives at them
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kLoadWarp) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            bool ok = true;
            int st = 0;
            uint32_t phase = 0;
            const CUtensorMap* mb = (EPI == kEpiSwiglu && rank == 1) ? &map_b2 : &map_b;
            for (int id = pair_id; ok && id < p.tiles; id += pairs) {
                const Tile t = get_tile(p, id, kNPerTile);
                const int a_row = t.m0 + int(rank) * BMC;
                const int b_row = EPI == kEpiSwiglu ? t.n0 : t.n0 + int(rank) * (BN / 2);
                for (int kk = 0; kk < p.k_iters; kk += kStepsPerStage) {
                    const int n = min(kStepsPerStage, p.k_iters - kk);
                    ok = mbar_wait(bar(kBarEmpty + st), phase ^ 1u, abort_flag, 0);
                    if (!ok) break;
                    if (leader) mbar_arrive_expect_tx(bar(kBarFull + st), uint32_t(2 * n) * kStepBytes);
                    const uint32_t full = map_to_cta(bar(kBarFull + st), 0);
                    for (int j = 0; j < n; ++j) {
                        const uint32_t a_dst = smem_base + st * kStageBytes + j * kStepBytes;
                        const int k0 = (kk + j) * BK;
                        if (A_KM) {
#pragma unroll
                            for (int i = 0; i < BMC / 64; ++i) tma2_load_3d(a_dst + i * (BK * 128), &map_a, full, a_row + 64 * i, k0, t.b);
                        } else {
                            tma2_load_3d(a_dst, &map_a, full, k0, a_row, t.b);
                        }
                        if (B_KN) {
#pragma unroll
                            for (int i = 0; i < BN / 2 / 64; ++i)
                                tma2_load_3d(a_dst + kABytes + i * (BK * 128), mb, full, b_row + 64 * i, k0, t.b);
                        } else {
                            tma2_load_3d(a_dst + kABytes, mb, full, k0, b_row, t.b);
                        }
                    }
                    if (++st == kStages) { st = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer (first CTA of the pair) --------------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc = instr_desc_f16(BF16 ? 1 : 0, 2 * BMC, BN, A_KM, B_KN);
            bool ok = true;
            int st = 0, local = 0;
            uint32_t phase = 0;
            for (int id = pair_id; ok && id < p.tiles; id += pairs) {
                const int buf = local & 1;
                // both CTAs' epilogues have read this accumulator's previous tile
                ok = mbar_wait(bar(kBarAccEmpty + buf), ((local >> 1) & 1) ^ 1u, abort_flag, 1);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tm = tmem + buf * BN;
                for (int kk = 0; kk < p.k_iters; kk += kStepsPerStage) {
                    const int n = min(kStepsPerStage, p.k_iters - kk);
                    ok = mbar_wait(bar(kBarFull + st), phase, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (int j = 0; j < n; ++j) {
                        const uint32_t a_addr = smem_base + st * kStageBytes + j * kStepBytes;
                        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                        for (int ks = 0; ks < BK / 16; ++ks) {
                            const uint64_t a_desc = A_KM ? smem_desc_sw128(a_addr + ks * 16 * 128, BK * 128, 1024)
                                                         : smem_desc_sw128(a_addr + ks * 32, 16, 1024);
                            const uint64_t b_desc = B_KN ? smem_desc_sw128(b_addr + ks * 16 * 128, BK * 128, 1024)
                                                         : smem_desc_sw128(b_addr + ks * 32, 16, 1024);
                            mma2_ss(d_tm, a_desc, b_desc, idesc, (kk || j || ks) ? 1u : 0u);
                        }
                    }
                    // the stage is free in both CTAs once these MMAs have read it
                    tc_commit2(bar(kBarEmpty + st));
                    tc_commit2(map_to_cta(bar(kBarEmpty + st), 1));
                    if (++st == kStages) { st = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit2(bar(kBarAccFull + buf));
                tc_commit2(map_to_cta(bar(kBarAccFull + buf), 1));
                ++local;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue (both CTAs, own 128 rows) ---------------------
        const int wq = warp & 3;
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        const uint32_t stage0 = smem_base + kSmemOut + wq * 2 * kOutStage;
        bool ok = true;
        int local = 0;
        uint32_t nstore = 0;
        for (int id = pair_id; ok && id < p.tiles; id += pairs) {
            const Tile t = get_tile(p, id, kNPerTile);
            const int buf = local & 1;
            const int row_w = t.m0 + int(rank) * BMC + wq * 32;
            constexpr int kChunks = kNPerTile / 64;
            float stat = 0.f;
            if (EPI == kEpiRowScale) stat = __ldg(p.row_scale + int64_t(t.b) * p.M + min(row_w + lane, p.M - 1));
            ok = mbar_wait<32>(bar(kBarAccFull + buf), (local >> 1) & 1, abort_flag, 3);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem + lane_base + buf * BN;
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c) {
                uint32_t out[32];
                if (EPI == kEpiSwiglu) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t g[32], u[32];
                        tmem_ld32(acc + 64 * c + 32 * h, g);
                        tmem_ld32(acc + BN / 2 + 64 * c + 32 * h, u);
                        tmem_wait_ld();
                        tmem_ld_fence32(g);
                        tmem_ld_fence32(u);
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float r[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float gg = round16<BF16>(__uint_as_float(g[i + e]));
                                const float uu = round16<BF16>(__uint_as_float(u[i + e]));
                                r[e] = gg / (1.0f + __expf(-gg)) * uu;
                            }
                            out[16 * h + i / 2] = pack16<BF16>(r[0], r[1]);
                        }
                    }
                } else {
                    uint32_t o[64];
                    tmem_ld32(acc + 64 * c, reinterpret_cast<uint32_t(&)[32]>(o[0]));
                    tmem_ld32(acc + 64 * c + 32, reinterpret_cast<uint32_t(&)[32]>(o[32]));
                    tmem_wait_ld();
                    tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(o[0]));
                    tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(o[32]));
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        float x0 = __uint_as_float(o[i]), x1 = __uint_as_float(o[i + 1]);
                        if (EPI == kEpiRowScale) {
                            x0 *= stat;
                            x1 *= stat;
                        }
                        if (EPI == kEpiBias) {
                            const int col = t.n0 + 64 * c + i;
                            const uint16_t* bias = static_cast<const uint16_t*>(p.bias);
                            if (col < p.N) x0 += from16<BF16>(bias[col]);
                            if (col + 1 < p.N) x1 += from16<BF16>(bias[col + 1]);
                        }
                        out[i / 2] = pack16<BF16>(x0, x1);
                    }
                }
                if (c + 1 == kChunks) {
                    // the accumulator is in registers: the issuing thread may start the tile after next
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(bar(kBarAccEmpty + buf), 0));
                }
                const uint32_t stage = stage0 + (nstore & 1u) * kOutStage;
                if (lane == 0) tma_store_wait_read_but_last();
                __syncwarp();
#pragma unroll
                for (int v = 0; v < 8; ++v)
                    st_shared_v4(stage + lane * 128 + ((v ^ (lane & 7)) << 4),
                                 make_uint4(out[4 * v], out[4 * v + 1], out[4 * v + 2], out[4 * v + 3]));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (row_w < p.M && t.n0 + 64 * c < p.N) tma_store_3d(&map_c, stage, t.n0 + 64 * c, row_w, t.b);
                    tma_store_commit();
                }
                ++nstore;
            }
            ++local;
        }
        if (lane == 0) tma_store_wait_read();
    }

    // ------------------------------ common exit ------------------------------------
    // Neither CTA may free its half of the pair's tensor memory, or leave while the other's loads and
    // commits can still arrive at its barriers, before both are through.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc2(tmem, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = *abort_flag;
        __threadfence_system();
    }
}

template <bool BF16, bool A_KM, bool B_KN, int EPI>
int launch2(Gpu* g, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mc,
            const Params& p, cudaStream_t s) {
    auto kernel = gemm_tc2_kernel<BF16, A_KM, B_KN, EPI>;
    PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const int pairs = std::min(p.tiles, sms / 2);
    kernel<<<dim3(unsigned(2 * pairs)), kThreads, kSmemTotal, s>>>(ma, mb, mb2, mc, p);
    PB_LAUNCH_CHECK("gemm_tc2_kernel");
    return PARAS_OK;
}

}  // namespace

// Shapes the pair kernel takes: either operand in either layout, any batch count, epilogue none / bias /
// row scale / SwiGLU (the epilogues as in gemm_tc.cu: A as [M, K] rows; SwiGLU two [F, K] weights), at least half a wave of 256 x 256 tiles (the single-CTA kernel would fill the same
// share of the GPU with its 128-row tiles; below that it splits K instead).  A 256 x 128 tile variant for
// outputs whose last round of tiles is mostly empty was measured and dropped: its MMAs run at two thirds
// of the wide tile's rate ([4096]^3: 1019 against 1440 TFLOP/s), more than the fuller round returns.
bool gemm_tc2_eligible(const Gpu* g, const paras_gemm_args* a) {
    if (a->epilogue != kEpiNone && a->epilogue != kEpiBias && a->epilogue != kEpiRowScale && a->epilogue != kEpiSwiglu)
        return false;
    if (a->a_layout == PARAS_GEMM_A_KM && a->epilogue != kEpiNone) return false;
    if (a->b_layout == PARAS_GEMM_B_KN && a->epilogue == kEpiSwiglu) return false;
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const int n_per_tile = a->epilogue == kEpiSwiglu ? BN / 2 : BN;
    const int64_t tiles = ((a->M + 2 * BMC - 1) / (2 * BMC)) * ((a->N + n_per_tile - 1) / n_per_tile) * a->batch;
    return tiles >= sms / 4 && a->K >= 4 * BK && a->N > BN / 2;
}

int gemm_tc2_run(Gpu* g, const paras_gemm_args* a, cudaStream_t s) {
    int st;
    CUtensorMap ma, mb, mb2, mc;
    const bool at = a->a_layout == PARAS_GEMM_A_KM, kn = a->b_layout == PARAS_GEMM_B_KN;
    st = at ? make_tensor_map_3d(&ma, a->a, a->dtype, a->M, a->K, a->batch, a->lda, a->stride_a, 64, BK)
            : make_tensor_map_3d(&ma, a->a, a->dtype, a->K, a->M, a->batch, a->lda, a->stride_a, BK, BMC);
    if (st != PARAS_OK) return st;
    st = kn ? make_tensor_map_3d(&mb, a->b, a->dtype, a->N, a->K, a->batch, a->ldb, a->stride_b, 64, BK)
            : make_tensor_map_3d(&mb, a->b, a->dtype, a->K, a->N, a->batch, a->ldb, a->stride_b, BK, BN / 2);
    if (st != PARAS_OK) return st;
    mb2 = mb;
    if (a->epilogue == kEpiSwiglu &&
        (st = make_tensor_map_3d(&mb2, a->b2, a->dtype, a->K, a->N, a->batch, a->ldb, a->stride_b, BK, BN / 2)) != PARAS_OK) return st;
    if ((st = make_tensor_map_3d(&mc, a->c, a->dtype, a->N, a->M, a->batch, a->ldc, a->stride_c, 64, 32)) != PARAS_OK) return st;
    const int n_per_tile = a->epilogue == kEpiSwiglu ? BN / 2 : BN;
    Params p{};
    p.M = int(a->M); p.N = int(a->N); p.K = int(a->K); p.batch = int(a->batch);
    p.tiles_m = int((a->M + 2 * BMC - 1) / (2 * BMC));
    p.tiles_n = int((a->N + n_per_tile - 1) / n_per_tile);
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * p.batch;
    if (tiles > INT32_MAX) return fail(PARAS_E_UNSUPPORTED, "paras gemm: too many tiles");
    p.tiles = int(tiles);
    p.k_iters = int((a->K + BK - 1) / BK);
    p.bias = a->bias;
    p.row_scale = a->row_scale;
    p.status = g->status_dev;
    const bool bf = a->dtype == PARAS_BF16;
#define PB_GO(AT, KN, E) (bf ? launch2<true, AT, KN, E>(g, ma, mb, mb2, mc, p, s) : launch2<false, AT, KN, E>(g, ma, mb, mb2, mc, p, s))
    if (at) return kn ? PB_GO(true, true, kEpiNone) : PB_GO(true, false, kEpiNone);
    if (kn) {
        switch (a->epilogue) {
            case kEpiBias: return PB_GO(false, true, kEpiBias);
            case kEpiRowScale: return PB_GO(false, true, kEpiRowScale);
            default: return PB_GO(false, true, kEpiNone);
        }
    }
    switch (a->epilogue) {
        case kEpiBias: return PB_GO(false, false, kEpiBias);
        case kEpiSwiglu: return PB_GO(false, false, kEpiSwiglu);
        case kEpiRowScale: return PB_GO(false, false, kEpiRowScale);
        default: return PB_GO(false, false, kEpiNone);
    }
#undef PB_GO
}

}  // namespace pb
