// The projections of a decode step: C[M, N] = X[M, K] * W[N, K]^T (+ bias) with M, the number of tokens
// in flight, at most 256.  Same call sites as gemm_tc.cu (aten::linear / addmm of the reference,
// csrc/ops/vision_ops.cpp:248-309, 388-423); this kernel takes the calls whose cost is reading W once.
//
// The operands swap roles: a CTA computes D = W_tile * X^T, 128 weight rows on the MMA's M side and the
// tokens (padded to a multiple of 16) on its N side, so every byte a stage loads for the wide operand is
// weight, and the 192 KB ring holds 8 stages = 128 KB of weight in flight per SM.  A 128 x 256 tile of
// the general kernel moves 16 KB of (mostly padding) X rows per 32 KB of weight and has to split K across
// launches to fill the GPU.
//
// K is split inside a cluster instead: the S CTAs of a cluster (S = 1..8, chosen so that weight-row blocks
// x S fills the SMs) take consecutive K ranges of the same 128 weight rows, leave their fp32 partial tile
// in their own shared memory, and after a cluster barrier CTA r sums, for the tokens m = r, r + S, ...,
// the S partials through distributed shared memory, adds the bias, rounds once and stores C[m, n0 .. n0+127]
// (256 contiguous bytes).  One launch, no scratch in global memory, the same bits on every run.
//
// Roles (192 threads): warps 0-3 read the accumulator (a lane per weight row) and do the reduction, warp 4
// allocates TMEM and issues the MMAs, warp 5 is the TMA producer.  Every mbarrier wait is bounded.
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

constexpr int BW = 128;                 // weight rows per CTA (MMA M)
constexpr int BK = 64;
constexpr int kWBytes = BW * BK * 2;    // 16 KB
constexpr int kMaxTokens = 256;
constexpr int kRingBytes = 192 * 1024;   // one CTA per SM; half of it when the blocks need more than one round of CTAs
constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 4, kMmaWarp = 4, kLoadWarp = 5, kThreads = 192;
// shared memory: [barriers, TMEM base word, abort flag: 1 KB][ring]
constexpr int kBarFull = 0, kBarEmpty = kMaxStages, kBarAccFull = 2 * kMaxStages;
constexpr int kNumBars = 2 * kMaxStages + 1;
constexpr int kSmemMisc = kNumBars * 8;
constexpr int kSmemRing = 1024;
constexpr int kMaxSplit = 8;

struct Params {
    int M, N, K;
    int tokens;        // M rounded up to a multiple of 16: the MMA's N
    int stages;
    int stage_bytes;   // kWBytes + tokens * 128
    int k_iters;       // K steps of 64 in all
    int tmem_cols;
    const void* bias;
    const float* row_scale;   // C[m, :] *= row_scale[m] (RMSNorm folded into the projection), or null
    void* c;
    int64_t ldc;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_v4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
    return v;
}

// SWIGLU: a block is 64 features; its weight tile is 64 gate-weight rows over 64 up-weight rows (two
// loads), and the finishing step forms silu(gate) * up from the two halves of a token's partial sums,
// each rounded to the tensors' dtype first as two separate projections would leave them
// (the reference's paras::swiglu_linear, csrc/ops/rms_swiglu_ops.cpp:77-104).
template <bool BF16, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    const uint32_t ring = smem_base + kSmemRing;
    auto bar = [&](int i) { return smem_base + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + kSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + kSmemMisc + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(), split = cluster_nctarank();
    const int n0 = int(blockIdx.x / split) * (SWIGLU ? BW / 2 : BW);
    // this CTA's K steps: the k_iters are dealt out in consecutive, nearly equal ranges
    const int per = p.k_iters / int(split), extra = p.k_iters % int(split);
    const int k_begin = int(rank) * per + min(int(rank), extra);
    const int k_count = per + (int(rank) < extra ? 1 : 0);

    if (smem_base & 1023u) {   // (the same in every CTA of the grid)
        if (threadIdx.x == 0) {
            *p.status = int(0x40000000u | (1u << 29));
            __threadfence_system();
        }
        return;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i) mbar_init(bar(i), 1u);
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_base + kSmemMisc, uint32_t(p.tmem_cols));
        tmem_relinquish();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_w);
        if (SWIGLU) tma_prefetch_desc(&map_w2);
        tma_prefetch_desc(&map_x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kLoadWarp) {
        if (lane == 0) {
            bool ok = true;
            int st = 0;
            uint32_t phase = 0;
            for (int i = 0; ok && i < k_count; ++i) {
                ok = mbar_wait(bar(kBarEmpty + st), phase ^ 1u, abort_flag, 0);
                if (!ok) break;
                const uint32_t full = bar(kBarFull + st);
                mbar_arrive_expect_tx(full, uint32_t(p.stage_bytes));
                const uint32_t dst = ring + st * p.stage_bytes;
                tma_load_3d(dst, &map_w, full, (k_begin + i) * BK, n0, 0);
                if (SWIGLU) tma_load_3d(dst + kWBytes / 2, &map_w2, full, (k_begin + i) * BK, n0, 0);
                tma_load_3d(dst + kWBytes, &map_x, full, (k_begin + i) * BK, 0, 0);
                if (++st == p.stages) { st = 0; phase ^= 1u; }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0 && k_count > 0) {
            const uint32_t idesc = instr_desc_f16(BF16 ? 1 : 0, BW, p.tokens, false, false);
            bool ok = true;
            int st = 0;
            uint32_t phase = 0;
            for (int i = 0; ok && i < k_count; ++i) {
                ok = mbar_wait(bar(kBarFull + st), phase, abort_flag, 2);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t w_addr = ring + st * p.stage_bytes;
                const uint32_t x_addr = w_addr + kWBytes;
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks)
                    mma_ss(tmem, smem_desc_sw128(w_addr + ks * 32, 16, 1024), smem_desc_sw128(x_addr + ks * 32, 16, 1024), idesc,
                           (i || ks) ? 1u : 0u);
                tc_commit(bar(kBarEmpty + st));
                if (++st == p.stages) { st = 0; phase ^= 1u; }
            }
            if (ok) tc_commit(bar(kBarAccFull));
        }
        __syncwarp();
    } else {
        // ---- the accumulator: lane = weight row, column = token -------------------------------
        const int row = warp * 32 + lane;                       // weight row within the tile
        float* part = reinterpret_cast<float*>(smem_raw + kSmemRing);   // [tokens][128] fp32, over the drained ring
        bool ok = true;
        if (k_count > 0) {
            ok = mbar_wait<32>(bar(kBarAccFull), 0, abort_flag, 3);
            if (ok) {
                tc_fence_after_sync();
                const uint32_t acc = tmem + (uint32_t(warp * 32) << 16);
                for (int c = 0; c < p.tokens; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(acc + c, v);
                    tmem_wait_ld();
                    tmem_ld_fence16(v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) part[(c + j) * BW + row] = __uint_as_float(v[j]);
                }
            }
        }
        if (!ok || k_count == 0)
            for (int c = 0; c < p.tokens; ++c) part[c * BW + row] = 0.f;   // (K shorter than the cluster: nothing to add)
        tc_fence_before_sync();
    }

    // every CTA's partial tile is in its shared memory
    __syncthreads();
    cluster_sync_all();
    if (SWIGLU && warp < kEpiWarps) {
        // half a warp per token: lane l of the half takes features 4l .. 4l+3, gate sums at [m][4l], up sums at [m][64 + 4l]
        const int l16 = lane & 15, half = lane >> 4;
        const int f = n0 + 4 * l16;
        uint32_t peer[kMaxSplit];
#pragma unroll
        for (int s2 = 0; s2 < kMaxSplit; ++s2) peer[s2] = map_to_cta(ring + uint32_t(l16) * 16u, uint32_t(s2) < split ? uint32_t(s2) : rank);
        const int mine = (p.M - int(rank) + int(split) - 1) / int(split);
        for (int i0 = 2 * warp + half; i0 < mine; i0 += 2 * kEpiWarps) {
            const int m = int(rank) + i0 * int(split);
            float4 v[2][kMaxSplit];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplit; ++s2)
                    v[u][s2] = uint32_t(s2) < split ? ld_cluster_v4(peer[s2] + uint32_t(m) * (BW * 4u) + uint32_t(u) * (BW * 2u))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplit; ++s2) {
                    acc[u][0] += v[u][s2].x; acc[u][1] += v[u][s2].y; acc[u][2] += v[u][s2].z; acc[u][3] += v[u][s2].w;
                }
            float r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float gg = round16<BF16>(acc[0][e]), uu = round16<BF16>(acc[1][e]);
                r[e] = gg / (1.0f + __expf(-gg)) * uu;
            }
            uint16_t* dst = static_cast<uint16_t*>(p.c) + int64_t(m) * p.ldc + f;
            const uint32_t lo = pack16<BF16>(r[0], r[1]), hi = pack16<BF16>(r[2], r[3]);
            if (f + 3 < p.N && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
            } else {
                if (f < p.N) dst[0] = uint16_t(lo & 0xffffu);
                if (f + 1 < p.N) dst[1] = uint16_t(lo >> 16);
                if (f + 2 < p.N) dst[2] = uint16_t(hi & 0xffffu);
                if (f + 3 < p.N) dst[3] = uint16_t(hi >> 16);
            }
        }
    } else if (warp < kEpiWarps) {
        // CTA `rank` finishes the tokens rank, rank + split, ...; a warp takes every fourth of them, a lane four
        // weight rows: 16-byte loads from each peer's tile, the loads of two tokens in flight before the first sum
        // (a remote load takes several hundred nanoseconds), an 8-byte store per lane = 256 contiguous bytes per warp.
        const int n = n0 + 4 * lane;
        uint32_t peer[kMaxSplit];
#pragma unroll
        for (int s2 = 0; s2 < kMaxSplit; ++s2) peer[s2] = map_to_cta(ring + uint32_t(lane) * 16u, uint32_t(s2) < split ? uint32_t(s2) : rank);
        float bias[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias)
            for (int e = 0; e < 4; ++e)
                if (n + e < p.N) bias[e] = from16<BF16>(static_cast<const uint16_t*>(p.bias)[n + e]);
        const int mine = (p.M - int(rank) + int(split) - 1) / int(split);   // tokens this CTA finishes
        for (int i0 = warp; i0 < mine; i0 += 2 * kEpiWarps) {
            float4 v[2][kMaxSplit];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int m = int(rank) + (i0 + u * kEpiWarps) * int(split);
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplit; ++s2)
                    v[u][s2] = (m < p.M && uint32_t(s2) < split) ? ld_cluster_v4(peer[s2] + uint32_t(m) * (BW * 4u))
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int m = int(rank) + (i0 + u * kEpiWarps) * int(split);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplit; ++s2) {   // fixed order: the same bits on every run
                    acc.x += v[u][s2].x; acc.y += v[u][s2].y; acc.z += v[u][s2].z; acc.w += v[u][s2].w;
                }
                if (m >= p.M) continue;
                if (p.row_scale) {
                    const float rs = __ldg(p.row_scale + m);
                    acc.x *= rs; acc.y *= rs; acc.z *= rs; acc.w *= rs;
                }
                uint16_t* dst = static_cast<uint16_t*>(p.c) + int64_t(m) * p.ldc + n;
                const uint32_t lo = pack16<BF16>(acc.x + bias[0], acc.y + bias[1]), hi = pack16<BF16>(acc.z + bias[2], acc.w + bias[3]);
                if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
                    *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
                } else {
                    if (n < p.N) dst[0] = uint16_t(lo & 0xffffu);
                    if (n + 1 < p.N) dst[1] = uint16_t(lo >> 16);
                    if (n + 2 < p.N) dst[2] = uint16_t(hi & 0xffffu);
                    if (n + 3 < p.N) dst[3] = uint16_t(hi >> 16);
                }
            }
        }
    }
    // no CTA leaves while another may still read its partial tile
    cluster_sync_all();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, uint32_t(p.tmem_cols));
    }
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = *abort_flag;
        __threadfence_system();
    }
}

}  // namespace

// X [M, K] rows with M <= 256, W [N, K] rows, one batch; no epilogue, a bias, a scale per row of X, or
// (M <= 128) the SwiGLU of two weights; K a multiple of 8 elements.
bool gemm_skinny_eligible(const Gpu* g, const paras_gemm_args* a) {
    if (a->a_layout != PARAS_GEMM_A_MK || a->b_layout != PARAS_GEMM_B_NK || a->batch != 1) return false;
    if (a->epilogue != 0 && a->epilogue != 1 && a->epilogue != 2 && a->epilogue != 5) return false;
    if (a->M > kMaxTokens || a->N < BW || a->K < 4 * BK) return false;
    if (a->epilogue == 2) return a->M <= 128;   // SwiGLU: 64 features per block, usually more blocks than SMs
    // more than 128 tokens leave room for one CTA per SM only: with more weight-row blocks than SMs the
    // second round of CTAs costs more than the general kernel's wider tiles ([256, 28672, 4096]: 89 against 60 us)
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    return a->M <= 128 || (a->N + BW - 1) / BW <= sms;
}

int gemm_skinny_run(Gpu* g, const paras_gemm_args* a, cudaStream_t s) {
    int st;
    Params p{};
    p.M = int(a->M); p.N = int(a->N); p.K = int(a->K);
    p.tokens = std::max(16, (p.M + 15) / 16 * 16);
    p.stage_bytes = kWBytes + p.tokens * 128;
    const int sms_all = g->sm_count > 0 ? g->sm_count : 148;
    const bool swiglu = a->epilogue == 2;
    const int rows_per_block = swiglu ? BW / 2 : BW;   // output columns a block produces
    const int blocks_all = int((a->N + rows_per_block - 1) / rows_per_block);
    // more weight-row blocks than SMs: half the ring, so that two CTAs share an SM and every block streams at once
    // (the partial tile of more than 128 tokens needs more than half the ring)
    const int ring_bytes = blocks_all > sms_all && p.tokens <= 128 ? kRingBytes / 2 : kRingBytes;
    const int smem_total = kSmemRing + ring_bytes;
    p.stages = std::min(kMaxStages, ring_bytes / p.stage_bytes);
    p.k_iters = (p.K + BK - 1) / BK;
    p.tmem_cols = p.tokens <= 32 ? 32 : p.tokens <= 64 ? 64 : p.tokens <= 128 ? 128 : 256;
    p.bias = a->epilogue == 1 ? a->bias : nullptr;
    p.row_scale = a->epilogue == 5 ? a->row_scale : nullptr;
    p.c = a->c;
    p.ldc = a->ldc;
    p.status = g->status_dev;
    CUtensorMap mw, mw2, mx;
    if ((st = make_tensor_map_3d(&mw, a->b, a->dtype, a->K, a->N, 1, a->ldb, a->stride_b, BK, rows_per_block)) != PARAS_OK) return st;
    mw2 = mw;
    if (swiglu && (st = make_tensor_map_3d(&mw2, a->b2, a->dtype, a->K, a->N, 1, a->ldb, a->stride_b, BK, rows_per_block)) != PARAS_OK) return st;
    if ((st = make_tensor_map_3d(&mx, a->a, a->dtype, a->K, a->M, 1, a->lda, a->stride_a, BK, p.tokens)) != PARAS_OK) return st;
    const int blocks = blocks_all;
    const bool bf = a->dtype == PARAS_BF16;
    const void* kernel = swiglu ? (bf ? (const void*)gemm_skinny_kernel<true, true> : (const void*)gemm_skinny_kernel<false, true>)
                                : (bf ? (const void*)gemm_skinny_kernel<true, false> : (const void*)gemm_skinny_kernel<false, false>);
    PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_total));
    // Split K so that as many SMs as possible stream weight at once, each CTA keeping at least 8 K steps.  How
    // many clusters of a size the GPU holds at a time depends on how its SMs group (a size that does not divide
    // a group leaves SMs out), so the driver is asked, once per size.
    constexpr int kGpuSlots = 64;
    static int fit[kGpuSlots][kMaxSplit + 1];   // clusters of size s resident at once; 0 = not asked yet
    // (asked with the plain kernel: both instantiations use the same shared memory and one CTA per SM here)
    int split = 1, best = std::min(blocks, g->sm_count > 0 ? g->sm_count : 148);
    for (int sz = 2; sz <= kMaxSplit && sz <= p.k_iters / 8 && blocks <= sms_all; ++sz) {
        int& f = fit[a->gpu % kGpuSlots][sz];
        if (f == 0) {
            cudaLaunchConfig_t q{};
            q.gridDim = dim3(unsigned(sz));
            q.blockDim = dim3(kThreads);
            q.dynamicSmemBytes = smem_total;
            cudaLaunchAttribute qa{};
            qa.id = cudaLaunchAttributeClusterDimension;
            qa.val.clusterDim.x = unsigned(sz); qa.val.clusterDim.y = 1; qa.val.clusterDim.z = 1;
            q.attrs = &qa;
            q.numAttrs = 1;
            int n = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &q);
            if (e != cudaSuccess) { cudaGetLastError(); n = -1; }
            f = n > 0 ? n : -1;
        }
        if (f < blocks) continue;               // would need a second round of clusters
        if (blocks * sz > best) { best = blocks * sz; split = sz; }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(blocks * split));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_total;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = unsigned(split);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    void* args[] = {(void*)&mw, (void*)&mw2, (void*)&mx, (void*)&p};
    PB_CUDA(cudaLaunchKernelExC(&cfg, kernel, args));
    return PARAS_OK;
}

}  // namespace pb
