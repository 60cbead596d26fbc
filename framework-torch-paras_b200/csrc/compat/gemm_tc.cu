// 16-bit GEMM for sm_100a with fp32 accumulation in TMEM: the projections on either side of
// the attention / RMSNorm / SwiGLU path (mm, bmm, addmm, linear: csrc/ops/vision_ops.cpp:
// 248-309, 388-423 hand these to the host's libtorch and copy the result back).
//
//   C[b][M,N] = A[b][M,K] * B[b]        A: [M,K] rows of K, or [K,M] rows of M (a transposed operand)
//                                       B: [N,K] rows of K (a Linear weight), or [K,N] rows of N
//   epilogues: none | + bias[N] | SwiGLU: C[M,F] = silu(A Wg^T) * (A Wu^T) from one pass over A
//              | * row_scale[M] (fp32): with B = W o w and row_scale = rstd this is RMSNorm(A) W^T,
//                the normalised activations never written (csrc/ops/rms_swiglu_ops.cpp:43-75 feeding
//                vision_ops.cpp:248-309)
//
// Persistent CTAs, one per SM, 128 x 256 output tiles, K in steps of 64:
//   warps 0-3  epilogue: TMEM -> registers -> 16 bit -> swizzled shared memory -> TMA store
//   warp  4    allocates TMEM; one lane issues tcgen05.mma (M128 x N256 x K16, 4 per K step)
//   warp  5    one lane issues the TMA loads: 4-stage ring of (A 16 KB, B 32 KB)
//   warps 6-9  (attention-backward epilogues only) a second epilogue group on every other 64 columns
// TMEM holds two 256-column accumulators, so the epilogue of a tile runs under the next
// tile's main loop.  For SwiGLU the B tile is 128 rows of the gate weight followed by 128
// rows of the up weight: one N=256 MMA leaves [gate | up] side by side in the accumulator.
// Tiles are taken in an order that keeps a 16 x 9 block of tiles (its A and B panels fit in
// L2 many times over) in flight at a time.
//
// Every wait is bounded (tc_prims.cuh); a wait that runs out raises the CTA's abort flag, all
// roles leave through the common exit, TMEM is freed and the GPU's status word is set.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "tc_prims.cuh"
#include "tma_host.cuh"
#include "gemm_internal.cuh"

namespace pb {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;         // 16 KB
constexpr int kBBytes = BN * BK * 2;         // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiWarps = 4;
constexpr int kMmaWarp = 4, kLoadWarp = 5;
constexpr int kThreads = 192;
// The attention-backward epilogues do per-element work on two-K-step tiles, so the epilogue is their
// critical path: those kernels run a second group of four epilogue warps (warps 6-9) that takes every
// other 64-column piece, and a three-stage ring whose fourth stage is the second group's staging.
constexpr int kThreadsWide = 320;
constexpr int kTmemCols = 512;               // two accumulators of BN columns
constexpr int kOutStage = 32 * 128;          // 32 rows x 64 columns of 16 bit
constexpr int kGroupM = 16;                  // tile order: 16 row blocks at a time

constexpr int kSmemOut = kStages * kStageBytes;                 // [4 warps][2] staging buffers
constexpr int kSmemBars = kSmemOut + kEpiWarps * 2 * kOutStage;
// With half-width B tiles a K step is 32 KB instead of 48 KB and its four MMAs take less time than the
// issuing thread needs per barrier round trip, so such a kernel moves two K steps per stage: the
// same 192 KB hold a ring of three 64 KB stages, and the waits and commits per byte halve.
constexpr int kNarrowStepBytes = kABytes + kBBytes / 2;
constexpr int kNarrowStageBytes = 2 * kNarrowStepBytes;
constexpr int kNarrowRing = kStages * kStageBytes / kNarrowStageBytes;   // 3
constexpr int kMaxRing = kStages;
constexpr int kBarFull = 0, kBarEmpty = kMaxRing, kBarAccFull = 2 * kMaxRing, kBarAccEmpty = 2 * kMaxRing + 2;
constexpr int kNumBars = 2 * kMaxRing + 4;
constexpr int kSmemMisc = kSmemBars + kNumBars * 8;             // tmem base word, abort flag
constexpr int kSmemTotal = kSmemMisc + 16;

enum { kEpiNone = 0, kEpiBias = 1, kEpiSwiglu = 2, kEpiProb = 3, kEpiDs = 4,   // 3, 4: attention backward only
       kEpiRowScale = 5,     // C = (A B^T) * row_scale[row]: RMSNorm folded into the projection that follows it
       kEpiPartial = 6 };    // split-K (internal): the fp32 accumulator itself, written through a 16-bit view of the buffer

struct GemmParams {
    int M, N, K;          // N = output columns (for SwiGLU: F)
    int batch;
    int tiles_m, tiles_n, tiles;   // per batch: tiles_m * tiles_n; tiles = all batches
    int k_iters;
    const void* bias;
    int* status;
    // attention backward epilogues (gemm_internal.cuh): per-row statistic, the probabilities, masking
    const float* row_stat;
    const void* prob;
    int64_t prob_ld;
    int Lq, causal;
    float scale, scale_log2;
    int k_skip;   // 0 none; 1: rows = queries, K = keys (dQ); 2: rows = keys, K = stacked queries (dV, dK)
    int tile_skip;  // rows = queries, columns = keys (P, dS): tiles with nothing visible are left alone
    int narrow;     // N <= 128: the B tile, the MMA and the epilogue cover 128 columns instead of 256
    int pair;       // causal reductions: tiles taken in heavy/light pairs (get_tile); the span they pair within
};

struct Tile { int b, m0, n0; };

// Causal reductions: a tile's work is the number of K steps it can see, which varies 16-fold with
// its row position.  There (p.pair, one column of tiles) ids 2i and 2i+1 are the i-th tile from the
// heavy end and the i-th from the light end of the same matrix (mode 2) or query head (mode 1), and a
// CTA takes both, so every CTA gets about the same work and both tiles read the same B operand.
__device__ __forceinline__ int first_tile(const GemmParams& p) { return p.pair ? 2 * int(blockIdx.x) : int(blockIdx.x); }
__device__ __forceinline__ int next_tile(const GemmParams& p, int id) {
    if (!p.pair) return id + int(gridDim.x);
    return (id & 1) ? id - 1 + 2 * int(gridDim.x) : id + 1;   // an odd count's last id + 1 ends the loop
}

__device__ __forceinline__ Tile get_tile(const GemmParams& p, int id, int n_per_tile) {
    const int per_batch = p.tiles_m * p.tiles_n;
    Tile t;
    if (p.pair) {
        t.b = id / p.tiles_m;
        const int q = id - t.b * p.tiles_m;
        const int span = p.pair;                 // tiles per matrix (mode 2) or per query head (mode 1)
        const int h = q / span, j = q - h * span;
        t.m0 = (h * span + ((j & 1) ? span - 1 - (j >> 1) : (j >> 1))) * BM;
        t.n0 = 0;
        return t;
    }
    t.b = id / per_batch;
    const int r = id - t.b * per_batch;
    const int in_group = kGroupM * p.tiles_n;
    const int group = r / in_group;
    const int first_m = group * kGroupM;
    const int gm = min(p.tiles_m - first_m, kGroupM);
    const int q = r - group * in_group;
    t.m0 = (first_m + q % gm) * BM;
    t.n0 = (q / gm) * n_per_tile;
    return t;
}

// The last query position among rows m0 .. m0+BM-1 of the stacked query heads (Lq rows each).
__device__ __forceinline__ int last_query_of_rows(const GemmParams& p, int m0) {
    const int q0 = m0 % p.Lq;
    return q0 + BM - 1 >= p.Lq ? p.Lq - 1 : q0 + BM - 1;
}

// Causal attention backward, P and dS: a tile all of whose keys come after all of its queries holds
// only zeros.  It is neither computed nor written; the products that read P and dS skip exactly
// those parts (skip_k_step), so what the memory holds there is never used.  All three roles apply
// the same test.
__device__ __forceinline__ bool skip_tile(const GemmParams& p, const Tile& t) {
    return p.tile_skip && t.n0 > last_query_of_rows(p, t.m0);
}

// Causal attention backward: K steps whose slice of P / dS is entirely masked contribute nothing.
// The same test runs in the loading and in the issuing thread.  With keys along K the first step
// is visible to every query, so an accumulator is always written; with queries along K the last
// step always runs, so that a key tile no query sees still gets a (zero) accumulator.
__device__ __forceinline__ bool skip_k_step(const GemmParams& p, int m0, int kk) {
    if (p.k_skip == 0) return false;
    if (p.k_skip == 1)  // rows m0.. are queries (stacked heads): keys from kk*BK on are masked for all of them?
        return kk * BK > last_query_of_rows(p, m0);
    if (kk + 1 == p.k_iters) return false;
    // rows m0.. are keys; the K step covers stacked queries kk*BK .. kk*BK+BK-1
    const int q0 = (kk * BK) % p.Lq;
    const int qmax = q0 + BK - 1 >= p.Lq ? p.Lq - 1 : q0 + BK - 1;
    return qmax < m0;
}

// The first K step at or after kk that runs (k_iters if none).
__device__ __forceinline__ int next_k_step(const GemmParams& p, int m0, int kk) {
    while (kk < p.k_iters && skip_k_step(p, m0, kk)) ++kk;
    return kk;
}

template <bool BF16, bool A_ROWS_OF_M, bool B_ROWS_OF_N, int EPI>
__global__ void __launch_bounds__((EPI == kEpiProb || EPI == kEpiDs) ? kThreadsWide : kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c,
               const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    auto bar = [&](int i) { return smem_base + kSmemBars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + kSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + kSmemMisc + 4);
    constexpr int kNPerTile = EPI == kEpiSwiglu ? BN / 2 : BN;   // output columns per tile
    constexpr bool kWide = EPI == kEpiProb || EPI == kEpiDs;
    constexpr int kEpiGroups = kWide ? 2 : 1;                    // groups of four epilogue warps
    constexpr int kRing = kWide ? kStages - 1 : kStages;          // stages of the operand ring in use

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (smem_base & 1023u) {
        // the 128-byte swizzle of TMA and of the MMA descriptors assumes 1024-byte aligned tiles
        if (threadIdx.x == 0) {
            *p.status = int(0x40000000u | (1u << 29));
            __threadfence_system();
        }
        return;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i)
            mbar_init(bar(i), i >= kBarAccEmpty ? uint32_t(kEpiWarps * kEpiGroups) : 1u);
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_base + kSmemMisc, kTmemCols);
        tmem_relinquish();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (EPI == kEpiSwiglu) tma_prefetch_desc(&map_b2);
        tma_prefetch_desc(&map_c);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kLoadWarp) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            bool ok = true;
            const int ring = p.narrow ? kNarrowRing : kRing;
            const uint32_t stage_bytes = p.narrow ? kNarrowStageBytes : kStageBytes;
            const uint32_t step_bytes = p.narrow ? kNarrowStepBytes : kStageBytes;
            int st = 0;            // ring position and its phase, across tiles
            uint32_t phase = 0;
            // full-width tiles: one K step per stage, constants known at compile time
            for (int id = first_tile(p); !p.narrow && ok && id < p.tiles; id = next_tile(p, id)) {
                const Tile t = get_tile(p, id, kNPerTile);
                if (skip_tile(p, t)) continue;
                for (int kk = 0; kk < p.k_iters; ++kk) {
                    if (skip_k_step(p, t.m0, kk)) continue;
                    ok = mbar_wait(bar(kBarEmpty + st), phase ^ 1u, abort_flag, 0);
                    if (!ok) break;
                    const uint32_t full = bar(kBarFull + st);
                    mbar_arrive_expect_tx(full, kStageBytes);
                    const uint32_t a_dst = smem_base + st * kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    if (A_ROWS_OF_M) {
#pragma unroll
                        for (int i = 0; i < BM / 64; ++i)
                            tma_load_3d(a_dst + i * (BK * 128), &map_a, full, t.m0 + 64 * i, kk * BK, t.b);
                    } else {
                        tma_load_3d(a_dst, &map_a, full, kk * BK, t.m0, t.b);
                    }
                    if (B_ROWS_OF_N) {
#pragma unroll
                        for (int i = 0; i < BN / 64; ++i)
                            tma_load_3d(b_dst + i * (BK * 128), &map_b, full, t.n0 + 64 * i, kk * BK, t.b);
                    } else if (EPI == kEpiSwiglu) {
                        tma_load_3d(b_dst, &map_b, full, kk * BK, t.n0, t.b);                // gate rows
                        tma_load_3d(b_dst + kBBytes / 2, &map_b2, full, kk * BK, t.n0, t.b);  // up rows
                    } else {
                        tma_load_3d(b_dst, &map_b, full, kk * BK, t.n0, t.b);
                    }
                    if (++st == kRing) { st = 0; phase ^= 1u; }
                }
            }
            // half-width tiles: two K steps per stage
            for (int id = first_tile(p); p.narrow && ok && id < p.tiles; id = next_tile(p, id)) {
                const Tile t = get_tile(p, id, kNPerTile);
                if (skip_tile(p, t)) continue;
                int kk = next_k_step(p, t.m0, 0);
                while (kk < p.k_iters) {
                    // the K steps of this stage: one, or (half-width tiles) the next two that run
                    int ks[2], n = 0;
                    ks[n++] = kk;
                    kk = next_k_step(p, t.m0, kk + 1);
                    if (p.narrow && kk < p.k_iters) {
                        ks[n++] = kk;
                        kk = next_k_step(p, t.m0, kk + 1);
                    }
                    ok = mbar_wait(bar(kBarEmpty + st), phase ^ 1u, abort_flag, 0);
                    if (!ok) break;
                    const uint32_t full = bar(kBarFull + st);
                    mbar_arrive_expect_tx(full, uint32_t(n) * step_bytes);
                    for (int j = 0; j < n; ++j) {
                        const int k0 = ks[j] * BK;
                        const uint32_t a_dst = smem_base + st * stage_bytes + j * step_bytes;
                        const uint32_t b_dst = a_dst + kABytes;
                        if (A_ROWS_OF_M) {
                            // A is [K, M]: two 64-row-of-M slabs of 64 K-rows each
#pragma unroll
                            for (int i = 0; i < BM / 64; ++i)
                                tma_load_3d(a_dst + i * (BK * 128), &map_a, full, t.m0 + 64 * i, k0, t.b);
                        } else {
                            tma_load_3d(a_dst, &map_a, full, k0, t.m0, t.b);
                        }
                        if (B_ROWS_OF_N) {
                            // B is [K, N]: four (narrow: two) 64-column slabs of 64 K-rows each
#pragma unroll
                            for (int i = 0; i < BN / 64; ++i)
                                if (i < 2 || !p.narrow)
                                    tma_load_3d(b_dst + i * (BK * 128), &map_b, full, t.n0 + 64 * i, k0, t.b);
                        } else if (EPI == kEpiSwiglu) {
                            tma_load_3d(b_dst, &map_b, full, k0, t.n0, t.b);                // gate rows
                            tma_load_3d(b_dst + kBBytes / 2, &map_b2, full, k0, t.n0, t.b);  // up rows
                        } else {
                            tma_load_3d(b_dst, &map_b, full, k0, t.n0, t.b);
                        }
                    }
                    if (++st == ring) { st = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = p.narrow ? instr_desc_f16(BF16 ? 1 : 0, BM, BN / 2, A_ROWS_OF_M, B_ROWS_OF_N)
                                            : instr_desc_f16(BF16 ? 1 : 0, BM, BN, A_ROWS_OF_M, B_ROWS_OF_N);
            bool ok = true;
            const int ring = p.narrow ? kNarrowRing : kRing;
            const uint32_t stage_bytes = p.narrow ? kNarrowStageBytes : kStageBytes;
            const uint32_t step_bytes = p.narrow ? kNarrowStepBytes : kStageBytes;
            int st = 0, local = 0;
            uint32_t phase = 0;
            for (int id = first_tile(p); ok && id < p.tiles; id = next_tile(p, id)) {
                Tile t{0, 0, 0};
                if (p.k_skip || p.tile_skip) {
                    t = get_tile(p, id, kNPerTile);
                    if (skip_tile(p, t)) continue;
                }
                const int buf = local & 1;
                // the epilogue has read this accumulator's previous tile
                ok = mbar_wait(bar(kBarAccEmpty + buf), ((local >> 1) & 1) ^ 1u, abort_flag, 1);
                if (!ok) break;
                const uint32_t d_tm = tmem + buf * BN;
                const int m0 = t.m0;
                bool first = true;  // the first K step that runs overwrites the accumulator
                // full-width tiles: one K step per stage
                for (int kk = 0; !p.narrow && kk < p.k_iters; ++kk) {
                    if (skip_k_step(p, m0, kk)) continue;
                    ok = mbar_wait(bar(kBarFull + st), phase, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_base + st * kStageBytes;
                    const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        const uint64_t a_desc = A_ROWS_OF_M
                            ? smem_desc_sw128(a_addr + ks * 16 * 128, BK * 128, 1024)
                            : smem_desc_sw128(a_addr + ks * 32, 16, 1024);
                        const uint64_t b_desc = B_ROWS_OF_N
                            ? smem_desc_sw128(b_addr + ks * 16 * 128, BK * 128, 1024)
                            : smem_desc_sw128(b_addr + ks * 32, 16, 1024);
                        mma_ss(d_tm, a_desc, b_desc, idesc, (!first || ks) ? 1u : 0u);
                    }
                    first = false;
                    tc_commit(bar(kBarEmpty + st));
                    if (++st == kRing) { st = 0; phase ^= 1u; }
                }
                // half-width tiles: two K steps per stage
                int kk = p.narrow ? next_k_step(p, m0, 0) : p.k_iters;
                while (kk < p.k_iters) {
                    // as in the loading thread: one K step per stage, or the next two that run
                    int n = 1;
                    kk = next_k_step(p, m0, kk + 1);
                    if (p.narrow && kk < p.k_iters) {
                        n = 2;
                        kk = next_k_step(p, m0, kk + 1);
                    }
                    ok = mbar_wait(bar(kBarFull + st), phase, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (int j = 0; j < n; ++j) {
                        const uint32_t a_addr = smem_base + st * stage_bytes + j * step_bytes;
                        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                        for (int ks = 0; ks < BK / 16; ++ks) {
                            const uint64_t a_desc = A_ROWS_OF_M
                                ? smem_desc_sw128(a_addr + ks * 16 * 128, BK * 128, 1024)
                                : smem_desc_sw128(a_addr + ks * 32, 16, 1024);
                            const uint64_t b_desc = B_ROWS_OF_N
                                ? smem_desc_sw128(b_addr + ks * 16 * 128, BK * 128, 1024)
                                : smem_desc_sw128(b_addr + ks * 32, 16, 1024);
                            mma_ss(d_tm, a_desc, b_desc, idesc, (!first || ks) ? 1u : 0u);
                        }
                        first = false;
                    }
                    tc_commit(bar(kBarEmpty + st));
                    if (++st == ring) { st = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(bar(kBarAccFull + buf));
                ++local;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue -----------------------------------
        const int wq = warp & 3;                 // TMEM lanes 32*wq .. 32*wq+31: a warp reaches its own quarter only
        const int eg = warp < kEpiWarps ? 0 : 1; // second group: warps 6-9, only in the wide kernels
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        const uint32_t stage0 = (eg == 0 ? smem_base + kSmemOut : smem_base + (kStages - 1) * kStageBytes) +
                                wq * 2 * kOutStage;
        bool ok = true;
        int local = 0;
        uint32_t nstore = 0;  // stores issued by this warp (picks the staging buffer)
        for (int id = first_tile(p); ok && id < p.tiles; id = next_tile(p, id)) {
            const Tile t = get_tile(p, id, kNPerTile);
            if (skip_tile(p, t)) continue;
            const int buf = local & 1;
            const int row_w = t.m0 + wq * 32;
            const int kChunks = p.narrow ? kNPerTile / 128 : kNPerTile / 64;  // 64 output columns per store
            // Attention-backward epilogues: a thread owns a row, so the row's statistic is one value per
            // thread.  It, and the first piece of P, are fetched before the wait for the accumulator, so
            // that their latency runs under the tile's main loop; the four epilogue warps have nothing
            // else to hide it behind.
            float stat = 0.f;
            int qpos = 0, qmin = 0, qmax = 0;
            const uint16_t* prow = nullptr;
            uint4 pcur[8];
            auto load_prob = [&](int c, uint4 (&dst)[8]) {
                const int col0 = t.n0 + 64 * c;
                const bool visible = !(p.causal && col0 > qmax);   // else every probability of the piece is zero
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    dst[v] = make_uint4(0, 0, 0, 0);
                    if (visible && col0 + 8 * v < p.N) dst[v] = __ldg(reinterpret_cast<const uint4*>(prow + col0) + v);
                }
            };
            if (EPI == kEpiRowScale) stat = __ldg(p.row_stat + int64_t(t.b) * p.M + min(row_w + lane, p.M - 1));
            if (EPI == kEpiProb || EPI == kEpiDs) {
                const int row = min(row_w + lane, p.M - 1);
                const int64_t grow = int64_t(t.b) * p.M + row;
                stat = __ldg(p.row_stat + grow);
                qpos = row % p.Lq;
                // whole 64-column pieces are usually either visible to all 32 rows or to none
                qmin = __reduce_min_sync(0xffffffffu, qpos);
                qmax = __reduce_max_sync(0xffffffffu, qpos);
                if (EPI == kEpiDs) {
                    prow = static_cast<const uint16_t*>(p.prob) + grow * p.prob_ld;
                    load_prob(eg, pcur);
                }
            }
            ok = mbar_wait<32>(bar(kBarAccFull + buf), (local >> 1) & 1, abort_flag, 3);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem + lane_base + buf * BN;
#pragma unroll 1
            for (int c = eg; c < kChunks; c += kEpiGroups) {
                uint32_t out[32];  // 64 outputs, packed in pairs
                uint4 pnext[8];
                if (EPI == kEpiDs && c + kEpiGroups < kChunks) load_prob(c + kEpiGroups, pnext);  // in flight during this piece
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
                            // the two projections are rounded to the tensor dtype as separate
                            // GEMMs would leave them; silu(g)*u is then rounded once
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
                    if (EPI == kEpiPartial) {
                        // 64 fp32 columns leave as two 128-byte-wide pieces; the tensor map sees each fp32 as two
                        // 16-bit elements, so a piece is the usual 64-element box at twice the column index
                        if (c + kEpiGroups >= kChunks) {
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar(kBarAccEmpty + buf));
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t stage = stage0 + (nstore & 1u) * kOutStage;
                            if (lane == 0) tma_store_wait_read_but_last();
                            __syncwarp();
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                st_shared_v4(stage + lane * 128 + ((v ^ (lane & 7)) << 4),
                                             make_uint4(o[32 * h + 4 * v], o[32 * h + 4 * v + 1], o[32 * h + 4 * v + 2],
                                                        o[32 * h + 4 * v + 3]));
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                if (row_w < p.M && t.n0 + 64 * c + 32 * h < p.N)
                                    tma_store_3d(&map_c, stage, 2 * (t.n0 + 64 * c + 32 * h), row_w, t.b);
                                tma_store_commit();
                            }
                            ++nstore;
                        }
                        continue;
                    }
                    if (EPI == kEpiProb) {
                        // C = exp(acc * scale - stat[row]), zero where the key comes after the query
                        const float neg = -stat * 1.4426950408889634f;
                        const int col0 = t.n0 + 64 * c;
                        if (!p.causal || col0 + 63 <= qmin) {
#pragma unroll
                            for (int i = 0; i < 64; ++i)
                                o[i] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(o[i]), p.scale_log2, neg)));
                        } else if (col0 > qmax) {
#pragma unroll
                            for (int i = 0; i < 64; ++i) o[i] = 0u;
                        } else {
#pragma unroll
                            for (int i = 0; i < 64; ++i)
                                o[i] = col0 + i <= qpos
                                           ? __float_as_uint(ex2_approx(fmaf(__uint_as_float(o[i]), p.scale_log2, neg)))
                                           : 0u;
                        }
                    } else if (EPI == kEpiDs) {
                        // C = P o (acc - stat[row]) * scale; P is zero where the key comes after the query
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const uint32_t ww[4] = {pcur[v].x, pcur[v].y, pcur[v].z, pcur[v].w};
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float pv = from16<BF16>(uint16_t((ww[e >> 1] >> (16 * (e & 1))) & 0xffffu));
                                o[8 * v + e] = __float_as_uint(pv * (__uint_as_float(o[8 * v + e]) - stat) * p.scale);
                            }
                        }
#pragma unroll
                        for (int v = 0; v < 8; ++v) pcur[v] = pnext[v];
                    }
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
                if (c + kEpiGroups >= kChunks) {
                    // the accumulator is in registers: the MMA warp may start the tile after next
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(kBarAccEmpty + buf));
                }
                const uint32_t stage = stage0 + (nstore & 1u) * kOutStage;
                if (lane == 0) tma_store_wait_read_but_last();  // the store before last has read this buffer
                __syncwarp();
#pragma unroll
                for (int v = 0; v < 8; ++v)
                    st_shared_v4(stage + lane * 128 + ((v ^ (lane & 7)) << 4),
                                 make_uint4(out[4 * v], out[4 * v + 1], out[4 * v + 2], out[4 * v + 3]));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (row_w < p.M && t.n0 + 64 * c < p.N)
                        tma_store_3d(&map_c, stage, t.n0 + 64 * c, row_w, t.b);
                    tma_store_commit();  // always: the waits above count groups
                }
                ++nstore;
            }
            ++local;
        }
        if (lane == 0) tma_store_wait_read();  // shared memory stays valid until the last store has read it
    }

    // ------------------------------ common exit ------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = *abort_flag;
        __threadfence_system();
    }
}

bool aligned16(const void* ptr, int64_t ld) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && ld % 8 == 0 && ld > 0;
}

// Split-K: C[m, n] = round(sum over the K slices of partial[s][m, n] (+ bias[n])), four columns per thread.
template <bool BF16>
__global__ void __launch_bounds__(256)
gemm_splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t M, int64_t N, const void* __restrict__ bias,
                          void* __restrict__ c, int64_t ldc) {
    const int64_t n4 = N / 4, total = M * n4;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int64_t m = i / n4, n = (i - m * n4) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sidx = 0; sidx < splits; ++sidx) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(partial + (int64_t(sidx) * M + m) * N + n));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (bias) {
            const uint16_t* bp = static_cast<const uint16_t*>(bias) + n;
            acc.x += from16<BF16>(bp[0]); acc.y += from16<BF16>(bp[1]); acc.z += from16<BF16>(bp[2]); acc.w += from16<BF16>(bp[3]);
        }
        uint2 o;
        o.x = pack16<BF16>(acc.x, acc.y);
        o.y = pack16<BF16>(acc.z, acc.w);
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(c) + m * ldc + n) = o;
    }
}

template <bool BF16, bool A_ROWS_OF_M, bool B_ROWS_OF_N, int EPI>
int launch(Gpu* g, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2,
           const CUtensorMap& mc, const GemmParams& p, cudaStream_t s) {
    auto kernel = gemm_tc_kernel<BF16, A_ROWS_OF_M, B_ROWS_OF_N, EPI>;
    PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const int units = p.pair ? (p.tiles + 1) / 2 : p.tiles;   // what a CTA takes per round
    kernel<<<dim3(unsigned(units < sms ? units : sms)), (EPI == kEpiProb || EPI == kEpiDs) ? kThreadsWide : kThreads, kSmemTotal, s>>>(
        ma, mb, mb2, mc, p);
    PB_LAUNCH_CHECK("gemm_tc_kernel");
    return PARAS_OK;
}

}  // namespace
}  // namespace pb

namespace pb {
int gemm_run(const paras_gemm_args* a, const GemmExtra* ex) {
    if (!a) return fail(PARAS_E_INVALID, "paras gemm: null args");
    if (a->dtype != PARAS_BF16 && a->dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras gemm: only 16-bit tensors run on the tensor-core kernel");
    if (a->M < 0 || a->N < 0 || a->K < 0 || a->batch < 0)
        return fail(PARAS_E_INVALID, "paras gemm: negative size");
    const int epi = ex ? ex->epilogue : a->epilogue;
    if ((a->epilogue < kEpiNone || a->epilogue > kEpiSwiglu) && a->epilogue != kEpiRowScale)
        return fail(PARAS_E_INVALID, "paras gemm: bad epilogue %d", a->epilogue);
    if (a->epilogue == kEpiRowScale && !a->row_scale)
        return fail(PARAS_E_INVALID, "paras gemm: row-scale epilogue without row_scale");
    if (ex && ex->epilogue != kEpiNone &&
        (a->a_layout != PARAS_GEMM_A_MK || (epi != kEpiProb && epi != kEpiDs) || !ex->row_stat ||
         (epi == kEpiDs && !ex->prob)))
        return fail(PARAS_E_INVALID, "paras gemm: bad internal epilogue request");
    if (a->b_layout != PARAS_GEMM_B_NK && a->b_layout != PARAS_GEMM_B_KN)
        return fail(PARAS_E_INVALID, "paras gemm: bad b_layout %d", a->b_layout);
    if (a->a_layout != PARAS_GEMM_A_MK && a->a_layout != PARAS_GEMM_A_KM)
        return fail(PARAS_E_INVALID, "paras gemm: bad a_layout %d", a->a_layout);
    if (a->a_layout == PARAS_GEMM_A_KM && a->epilogue != kEpiNone)
        return fail(PARAS_E_UNSUPPORTED, "paras gemm: epilogues take A as rows of K");
    int st;
    Gpu* g = use_gpu(a->gpu, &st);
    if (!g) return st;
    if (g->cc_major != 10) return fail(PARAS_E_UNSUPPORTED, "paras gemm: GPU is not compute capability 10.x");
    if (a->M == 0 || a->N == 0 || a->batch == 0) return PARAS_OK;
    if (a->K == 0) return fail(PARAS_E_UNSUPPORTED, "paras gemm: K = 0");
    if (a->M > INT32_MAX || a->N > INT32_MAX || a->K > INT32_MAX || a->batch > 65535)
        return fail(PARAS_E_UNSUPPORTED, "paras gemm: sizes exceed 32-bit tile coordinates");
    if (!a->a || !a->b || !a->c) return fail(PARAS_E_INVALID, "paras gemm: null pointer");
    if (a->epilogue == kEpiBias && !a->bias) return fail(PARAS_E_INVALID, "paras gemm: bias epilogue without bias");
    if (a->epilogue == kEpiSwiglu && (!a->b2 || a->b_layout != PARAS_GEMM_B_NK))
        return fail(PARAS_E_INVALID, "paras gemm: the SwiGLU epilogue takes two [F,K] weights");
    if (!aligned16(a->a, a->lda) || !aligned16(a->b, a->ldb) || !aligned16(a->c, a->ldc) ||
        (a->epilogue == kEpiSwiglu && !aligned16(a->b2, a->ldb)) ||
        (a->batch > 1 && (a->stride_a % 8 || a->stride_b % 8 || a->stride_c % 8)))
        return fail(PARAS_E_UNSUPPORTED, "paras gemm: pointers or strides are not 16-byte aligned");
    if (g->smem_optin < size_t(kSmemTotal)) return fail(PARAS_E_UNSUPPORTED, "paras gemm: not enough shared memory");
    if ((st = check_status_word(g)) != PARAS_OK) return st;

    const bool kn = a->b_layout == PARAS_GEMM_B_KN;
    const bool at = a->a_layout == PARAS_GEMM_A_KM;
    // N <= 128 (the [.., head dim] products of attention backward): half-width B tiles and MMAs
    const bool narrow = a->N <= BN / 2 && (epi == kEpiNone || epi == kEpiBias || epi == kEpiRowScale);
    const int n_per_tile = a->epilogue == kEpiSwiglu || narrow ? BN / 2 : BN;
    // A handful of rows against a weight: the weight-streaming kernel (PARAS_GEMM_SKINNY=0: this file's split-K)
    static const bool skinny_off = getenv("PARAS_GEMM_SKINNY") && getenv("PARAS_GEMM_SKINNY")[0] == '0';
    if (!ex && !skinny_off && gemm_skinny_eligible(g, a)) return gemm_skinny_run(g, a, pick_stream(g, a->stream));
    // Large projections run on CTA pairs (PARAS_GEMM_PAIR=0 keeps them on this file's kernel, for comparison)
    static const bool pair_off = getenv("PARAS_GEMM_PAIR") && getenv("PARAS_GEMM_PAIR")[0] == '0';
    if (!ex && !pair_off && gemm_tc2_eligible(g, a)) return gemm_tc2_run(g, a, pick_stream(g, a->stream));
    // Few output tiles and a long K (the projections of a decode step: M = the batch): the K range is cut
    // into slices that run as the batches of one launch, each writing its fp32 accumulator to scratch, and a
    // small kernel sums the slices, adds the bias and rounds.  Without it 16 of the 148 SMs stream the weight.
    if (!ex && !at && a->batch == 1 && (a->epilogue == kEpiNone || a->epilogue == kEpiBias) && a->N % 4 == 0) {
        const int sms = g->sm_count > 0 ? g->sm_count : 148;
        const int64_t tiles = ((a->M + BM - 1) / BM) * ((a->N + n_per_tile - 1) / n_per_tile);
        int splits = int(std::min<int64_t>(std::min<int64_t>(16, sms / std::max<int64_t>(tiles, 1)), a->K / (4 * BK)));
        while (splits > 1 && a->K % (int64_t(splits) * BK)) --splits;
        if (splits > 1) {
            const int64_t ks = a->K / splits;
            cudaStream_t s = pick_stream(g, a->stream);
            void* scratch = nullptr;
            if ((st = paras_b200_malloc_async(a->gpu, size_t(splits) * size_t(a->M) * size_t(a->N) * sizeof(float), s, &scratch)) != PARAS_OK)
                return st;
            CUtensorMap ma, mb, mc;
            st = make_tensor_map_3d(&ma, a->a, a->dtype, ks, a->M, splits, a->lda, ks, BK, BM);
            if (st == PARAS_OK)
                st = kn ? make_tensor_map_3d(&mb, a->b, a->dtype, a->N, ks, splits, a->ldb, ks * a->ldb, 64, BK)
                        : make_tensor_map_3d(&mb, a->b, a->dtype, ks, a->N, splits, a->ldb, ks, BK, n_per_tile);
            if (st == PARAS_OK)
                st = make_tensor_map_3d(&mc, scratch, a->dtype, 2 * a->N, a->M, splits, 2 * a->N, 2 * a->M * a->N, 64, 32);
            if (st == PARAS_OK) {
                GemmParams p{};
                p.M = int(a->M); p.N = int(a->N); p.K = int(ks); p.batch = splits;
                p.tiles_m = int((a->M + BM - 1) / BM);
                p.tiles_n = int((a->N + n_per_tile - 1) / n_per_tile);
                p.tiles = p.tiles_m * p.tiles_n * splits;
                p.k_iters = int(ks / BK);
                p.narrow = narrow;
                p.status = g->status_dev;
                const bool bf = a->dtype == PARAS_BF16;
                if (bf) st = kn ? launch<true, false, true, kEpiPartial>(g, ma, mb, mb, mc, p, s) : launch<true, false, false, kEpiPartial>(g, ma, mb, mb, mc, p, s);
                else st = kn ? launch<false, false, true, kEpiPartial>(g, ma, mb, mb, mc, p, s) : launch<false, false, false, kEpiPartial>(g, ma, mb, mb, mc, p, s);
                if (st == PARAS_OK) {
                    const int blocks = int(std::min<int64_t>((a->M * (a->N / 4) + 255) / 256, int64_t(sms) * 8));
                    const void* bias = a->epilogue == kEpiBias ? a->bias : nullptr;
                    if (bf) gemm_splitk_reduce_kernel<true><<<blocks, 256, 0, s>>>(static_cast<const float*>(scratch), splits, a->M, a->N, bias, a->c, a->ldc);
                    else gemm_splitk_reduce_kernel<false><<<blocks, 256, 0, s>>>(static_cast<const float*>(scratch), splits, a->M, a->N, bias, a->c, a->ldc);
                    if (cudaGetLastError() != cudaSuccess) st = fail(PARAS_E_CUDA, "paras gemm: split-K reduce launch failed");
                }
            }
            const int st2 = paras_b200_free_async(a->gpu, scratch, s);
            return st != PARAS_OK ? st : st2;
        }
    }
    CUtensorMap ma, mb, mb2, mc;
    if (at) {
        if ((st = make_tensor_map_3d(&ma, a->a, a->dtype, a->M, a->K, a->batch, a->lda, a->stride_a, 64, BK)) != PARAS_OK) return st;
    } else {
        if ((st = make_tensor_map_3d(&ma, a->a, a->dtype, a->K, a->M, a->batch, a->lda, a->stride_a, BK, BM)) != PARAS_OK) return st;
    }
    if (kn) {
        if ((st = make_tensor_map_3d(&mb, a->b, a->dtype, a->N, a->K, a->batch, a->ldb, a->stride_b, 64, BK)) != PARAS_OK) return st;
    } else {
        if ((st = make_tensor_map_3d(&mb, a->b, a->dtype, a->K, a->N, a->batch, a->ldb, a->stride_b, BK, n_per_tile)) != PARAS_OK) return st;
    }
    mb2 = mb;
    if (a->epilogue == kEpiSwiglu &&
        (st = make_tensor_map_3d(&mb2, a->b2, a->dtype, a->K, a->N, a->batch, a->ldb, a->stride_b, BK, n_per_tile)) != PARAS_OK) return st;
    if ((st = make_tensor_map_3d(&mc, a->c, a->dtype, a->N, a->M, a->batch, a->ldc, a->stride_c, 64, 32)) != PARAS_OK) return st;

    GemmParams p{};
    p.M = int(a->M); p.N = int(a->N); p.K = int(a->K); p.batch = int(a->batch);
    p.tiles_m = int((a->M + BM - 1) / BM);
    p.tiles_n = int((a->N + n_per_tile - 1) / n_per_tile);
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * p.batch;
    if (tiles > INT32_MAX) return fail(PARAS_E_UNSUPPORTED, "paras gemm: too many tiles");
    p.tiles = int(tiles);
    p.k_iters = int((a->K + BK - 1) / BK);
    p.narrow = narrow;
    p.bias = a->bias;
    p.row_stat = a->epilogue == kEpiRowScale ? a->row_scale : nullptr;
    p.status = g->status_dev;
    if (ex) {
        p.row_stat = ex->row_stat; p.prob = ex->prob; p.prob_ld = ex->prob_ld;
        p.Lq = ex->Lq > 0 ? ex->Lq : 1; p.causal = ex->causal; p.scale = ex->scale;
        p.scale_log2 = ex->scale * 1.4426950408889634f;
        p.k_skip = ex->causal ? ex->k_skip : 0;
        p.tile_skip = ex->causal && (epi == kEpiProb || epi == kEpiDs) ? ex->tile_skip : 0;
        if (p.k_skip == 2 && p.tiles_n == 1) p.pair = p.tiles_m;
        if (p.k_skip == 1 && p.tiles_n == 1 && p.Lq % BM == 0 && p.tiles_m % (p.Lq / BM) == 0) p.pair = p.Lq / BM;
    }
    cudaStream_t s = pick_stream(g, a->stream);
    const bool bf = a->dtype == PARAS_BF16;
#define PB_GEMM(AT, KN, EPI) (bf ? launch<true, AT, KN, EPI>(g, ma, mb, mb2, mc, p, s) : launch<false, AT, KN, EPI>(g, ma, mb, mb2, mc, p, s))
    if (epi == kEpiProb) return kn ? PB_GEMM(false, true, kEpiProb) : PB_GEMM(false, false, kEpiProb);
    if (epi == kEpiDs) return kn ? PB_GEMM(false, true, kEpiDs) : PB_GEMM(false, false, kEpiDs);
    if (a->epilogue == kEpiSwiglu) return PB_GEMM(false, false, kEpiSwiglu);
    if (a->epilogue == kEpiBias) return kn ? PB_GEMM(false, true, kEpiBias) : PB_GEMM(false, false, kEpiBias);
    if (a->epilogue == kEpiRowScale) return kn ? PB_GEMM(false, true, kEpiRowScale) : PB_GEMM(false, false, kEpiRowScale);
    if (at) return kn ? PB_GEMM(true, true, kEpiNone) : PB_GEMM(true, false, kEpiNone);
    return kn ? PB_GEMM(false, true, kEpiNone) : PB_GEMM(false, false, kEpiNone);
#undef PB_GEMM
}
}  // namespace pb

extern "C" int paras_b200_gemm(const paras_gemm_args* a) {
    pb::NvtxRange range("paras_b200_gemm");
    return pb::gemm_run(a, nullptr);
}
