// Fused flash-attention backward for sm_100a: tcgen05 tensor cores, TMEM accumulators, TMA.
//
// The gradient the reference obtains by autograd through its composite sdpa_math
// (csrc/ops/attention_ops.cpp:71-136) and its softmax backward (csrc/ops/pointwise_ops.cpp:
// 994-1062), without ever forming a [Lq, Lk] matrix in memory: the probabilities are rebuilt
// tile by tile from the forward's row statistics,
//
//     P  = exp(S * scale - lse[q])            S  = Q K^T
//     dS = P o (dP - delta[q]) * scale        dP = dO V^T,  delta[q] = sum_d dO[q,d] O[q,d]
//     dV = P^T dO      dK = dS^T Q      dQ = dS K
//
// Two kernels, each a persistent grid of one 352-thread CTA per SM, neither with atomics nor
// with scratch beyond the row statistic delta (so the result is deterministic):
//
//   sdpa_bwd_dq_kernel    (runs first) a CTA keeps one 128-query tile (Q_i, dO_i) in shared memory and
//       streams the key tiles it sees; S and dP land in TMEM with one QUERY per lane, dS goes back
//       to TMEM as the 16-bit A operand of dQ += dS K_j.  It also forms delta for its rows and writes
//       it out for the second kernel.
//   sdpa_bwd_dkv_kernel   the mirror image: a CTA keeps one 128-key tile (K_j, V_j) and streams
//       the query tiles that see it (all query heads of the kv head's group, so GQA sums happen
//       in the accumulator).  S^T = K_j Q_i^T and dP^T = V_j dO_i^T land with one KEY per lane;
//       P^T and dS^T go back to TMEM as the A operands of dV += P^T dO_i, dK += dS^T Q_i.
//
// S and dP are computed twice (7 tile products instead of 5) in exchange for no fp32 dQ
// accumulator in memory, no atomics and no conversion pass.
//
//   warps 0-3  element-wise work on one half of the columns of the S / dP tiles (a lane owns a row)
//   warps 4-7  the same on the other half
//   warp  8    one lane issues the products that form S and dP (S^T and dP^T)
//   warp  9    TMA loads (and, for the dK/dV kernel, the per-query statistics of each step)
//   warp 10    one lane issues the products that accumulate (dQ; dV and dK)
//
// Every wait is bounded (tc_prims.cuh): a wait that runs out raises the CTA's abort flag, all
// roles leave through the common exit, TMEM is freed and the GPU's status word is set.
#include <cmath>

#include "sdpa_common.cuh"
#include "tc_prims.cuh"
#include "tma_host.cuh"

namespace pb {
namespace {

using namespace tc;

constexpr int BT = 128;                       // rows of every tile: queries or keys
constexpr int kChunkBytes = 64 * 2 * 128;     // one 64-element slab of 128 rows
constexpr int kTileBytes = 2 * kChunkBytes;   // 128 x 128 x 2 B (head dim 64 uses the first slab)
constexpr int kMmaWarp = 8, kLoadWarp = 9;
constexpr int kTmemCols = 512;

constexpr int kSmemOwn = 0;                   // shared memory starts with the CTA's own pair: tile 0, tile 1

// The dQ kernel streams K and V through rings of their own: V_j is done with after dP = dO V_j^T,
// K_j only after dQ += dS K_j at the end of the step, so K gets three stages and V two (with one
// two-stage ring for the pair, every step waited about 1300 cycles for a load that could only
// start once the step before last had released its stage).
constexpr int kDqKStages = 3, kDqVStages = 2;
constexpr int kDqSmemK = 2 * kTileBytes;
constexpr int kDqSmemV = kDqSmemK + kDqKStages * kTileBytes;
constexpr int kDqSmemBars = kDqSmemV + kDqVStages * kTileBytes;
// One "landed" barrier per step for K_j and V_j together (two arrivals, each with its tile's bytes):
// an issuing thread's wait costs it a few hundred cycles even when the barrier completed long ago,
// because it is one thread between two busy warps of its scheduler.  Six of them, the least common
// multiple of the two ring depths, so that a barrier is never re-armed before its step is over.
constexpr int kDqFullBars = 6;
constexpr int kDqBarOwnFull = 0, kDqBarOwnEmpty = 1, kDqBarStepFull = 2 /* [6] */, kDqBarKEmpty = 8 /* [3] */,
              kDqBarVEmpty = 11 /* [2] */, kDqBarDpFull = 13, kDqBarTaken = 14, kDqBarDsFull = 15,
              kDqBarAccFull = 16, kDqBarAccEmpty = 17, kDqBarDsFree = 18 /* [2] */, kDqNumBars = 20;
constexpr int kDqSmemMisc = kDqSmemBars + kDqNumBars * 8;
constexpr int kDqSmemDelta = kDqSmemMisc + 16;            // fp32 [128]: delta of the item's rows
constexpr int kDqSmemLaunch = kDqSmemDelta + BT * 4 + 1024;

struct BwdParams {
    void* dq;
    void* dk;
    void* dv;
    const float* lse;     // [B, Hq, Lq]
    // Per-query statistics in the form the dK/dV kernel adds them, [B, Hq, nq * 128] (rows padded to whole
    // query tiles, so that 128-bit loads need no bounds): nlse2 = -lse * log2(e) (-inf past the last query:
    // its probabilities are 0) and nds = -delta * scale with delta = rowsum(dO o O) (0 past the last query).
    // Written by the dQ kernel for the rows of each of its items, read by the dK/dV kernel.
    float* nlse2;
    float* nds;
    const void* out;      // the forward's output and its gradient, dense [B, Hq, Lq, D] (for delta)
    const void* dout;
    int B, Hq, Hkv, Lq, Lk;
    int causal;
    float scale;
    float scale_log2;     // scale * log2(e)
    int* status;
    int nq, nk;           // 128-row tiles of queries / keys
    int npair;            // paired tiles per head (ceil(n / 2))
    int units;
};

// Query tiles that see key tile j, as the range [first, nq): under the top-left aligned causal
// mask query row r sees keys 0..r, so tile i qualifies when its last row reaches the tile's
// first key.
__device__ __forceinline__ int first_query_tile(const BwdParams& p, int j) {
    return p.causal ? min(j, p.nq) : 0;
}
// Key tiles query tile i sees: [0, n).
__device__ __forceinline__ int key_tiles_for(const BwdParams& p, int i) {
    int last = p.Lk;
    if (p.causal) last = min(last, min(p.Lq, (i + 1) * BT));
    return (last + BT - 1) / BT;
}

// One work item = one 128-row tile of the CTA's own pair: a key tile of one (batch, kv head) for
// the dK/dV kernel, a query tile of one (batch, query head) for the dQ kernel.  A unit pairs tiles
// (n-1-pair) and (pair) of one head: under a causal mask their work adds up to the same total for
// every pair, so handing out units round-robin keeps the persistent CTAs balanced.
struct Item {
    int b, h;   // batch, head of the own tile (kv head / query head)
    int t;      // tile index
    int n;      // streamed tiles (iterations); 0 = nothing streams (the outputs are zeros)
};

template <bool DKV>
__device__ __forceinline__ bool get_item(const BwdParams& p, int seq, Item* it) {
    const int unit = int(blockIdx.x) + (seq >> 1) * int(gridDim.x);
    if (unit >= p.units) return false;
    const int heads = DKV ? p.Hkv : p.Hq;
    const int tiles = DKV ? p.nk : p.nq;
    const int hb = unit / p.npair;
    const int pair = unit - hb * p.npair;
    const int hi = tiles - 1 - pair;
    it->b = hb / heads;
    it->h = hb - it->b * heads;
    it->t = (seq & 1) ? pair : hi;
    const bool dup = (seq & 1) && pair == hi;   // odd tile count: the middle tile has no partner
    if (dup) {
        it->n = -1;                              // not an item at all
    } else if (DKV) {
        it->n = (p.Hq / p.Hkv) * (p.nq - first_query_tile(p, it->t));
    } else {
        it->n = key_tiles_for(p, it->t);
    }
    return true;
}

// Stores 32 fp32 accumulator columns of this lane's row as 16-bit values: 64 contiguous bytes.
template <bool BF16>
__device__ __forceinline__ void store_row32(void* dst, const uint32_t (&o)[32]) {
    uint4* d = static_cast<uint4*>(dst);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        uint4 w;
        w.x = pack16<BF16>(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
        w.y = pack16<BF16>(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
        w.z = pack16<BF16>(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
        w.w = pack16<BF16>(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
        d[v] = w;
    }
}

// ---------------------------------------------------------------------------------------------
// dK / dV: own pair = (K_j, V_j), streamed = (Q, dO) of the query tiles that see the keys, 64
// queries per step, over the group's query heads.
//
// A step's chain is  S^T ready -> exponentials -> P^T handed back -> dV,  and with whole 128-query
// tiles that chain was the step: P^T overlays S^T in TMEM, so the next S^T had to wait for dV.  With
// 64 queries per step S^T and dP^T are 64 columns each and fit twice: the tensor core forms step
// x+1's pair in the other buffer while the element-wise warps work on step x, and the same shared
// memory holds a ring of four 64-query stages instead of two 128-query ones.
//
// Two threads issue MMAs, from different warps: one forms the (S^T, dP^T) pairs as soon as a ring
// stage and a TMEM buffer are free, the other issues dV and dK when the element-wise warps hand
// P^T and dS^T back.  An issuing thread is serial -- every wait costs it a few hundred cycles
// during which it issues nothing -- so with a single one the tensor core idled through each wait;
// the two streams wait on different things and keep it fed.
// ---------------------------------------------------------------------------------------------
constexpr int kDkvHalf = 64;                          // queries per step
constexpr int kDkvStages = 4;
constexpr int kDkvHalfChunkBytes = kDkvHalf * 128;    // one 64-column slab of 64 rows
constexpr int kDkvHalfTileBytes = 2 * kDkvHalfChunkBytes;
constexpr int kDkvStageBytes = 2 * kDkvHalfTileBytes; // Q half tile, dO half tile
constexpr int kDkvSmemRing = 2 * kTileBytes;
constexpr int kDkvSmemBars = kDkvSmemRing + kDkvStages * kDkvStageBytes;
constexpr int kDkvBarOwnFull = 0, kDkvBarOwnEmpty = 1, kDkvBarRingFull = 2, kDkvBarRingEmpty = 6,
              kDkvBarSFull = 10,    // [2] MMA -> compute: S^T in buffer b
              kDkvBarDpFull = 12,   // [2] MMA -> compute: dP^T in buffer b
              kDkvBarPFull = 14,    // compute -> MMA: P^T stored
              kDkvBarDsFull = 15,   // compute -> MMA: dS^T stored
              kDkvBarAccFull = 16, kDkvBarAccEmpty = 17,
              kDkvBarBufFree = 18,  // [2] accumulating issuer -> pair issuer: buffer b's P^T and dS^T are consumed
              kDkvNumBars = 20;
constexpr int kDkvThreads = 352;     // 8 element-wise warps, pair issuer, loader, accumulating issuer
constexpr int kAccWarp = 10;
constexpr int kDkvSmemMisc = kDkvSmemBars + kDkvNumBars * 8;
constexpr int kDkvSmemLaunch = kDkvSmemMisc + 16 + 1024;

template <bool BF16, int HD>
__global__ void __launch_bounds__(kDkvThreads, 1)
sdpa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto bar = [&](int i) { return smem_base + kDkvSmemBars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kDkvSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kDkvSmemMisc + 4);
    constexpr int kChunks = HD / 64;
    constexpr uint32_t kOwnBytes = kChunks * kChunkBytes;            // K_j or V_j
    constexpr uint32_t kHalfBytes = kChunks * kDkvHalfChunkBytes;    // 64 rows of Q or dO
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = p.Hq / p.Hkv;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kDkvNumBars; ++i) {
            const bool eight = i == kDkvBarPFull || i == kDkvBarDsFull || i == kDkvBarAccEmpty;
            mbar_init(bar(i), eight ? 8u : 1u);   // one arrival per compute warp / one commit or TMA
        }
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_base + kDkvSmemMisc, kTmemCols);
        tmem_relinquish();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // TMEM: S^T buffers @0, @64; dP^T buffers @128, @192; dV @256; dK @384
    constexpr int kColS = 0, kColDp = 128, kColDv = 256, kColDk = 384;

    // Step x of an item: query head hh of the group, query tile i, half (0 / 1) of the tile.
    // steps = 2 * (group size) * (query tiles that see the key tile)
    if (warp == kLoadWarp) {
        // ------------------------------ loads ------------------------------------------------
        bool ok = true;
        uint32_t items = 0, rc = 0;   // items loaded, ring stages filled
        Item it;
        for (int seq = 0; ok && get_item<true>(p, seq, &it); ++seq) {
            if (it.n <= 0) continue;
            if (lane == 0) {
                ok = mbar_wait(bar(kDkvBarOwnEmpty), (items & 1u) ^ 1u, abort_flag, 0);
                if (ok) {
                    mbar_arrive_expect_tx(bar(kDkvBarOwnFull), 2 * kOwnBytes);
#pragma unroll
                    for (int c = 0; c < kChunks; ++c) {
                        tma_load_4d(smem_base + kSmemOwn + c * kChunkBytes, &map_k, bar(kDkvBarOwnFull), 64 * c, it.t * BT, it.h, it.b);
                        tma_load_4d(smem_base + kSmemOwn + kTileBytes + c * kChunkBytes, &map_v, bar(kDkvBarOwnFull), 64 * c, it.t * BT, it.h, it.b);
                    }
                }
            }
            ++items;
            const int i0 = first_query_tile(p, it.t), cnt = 2 * (p.nq - i0);   // half tiles per query head
            const int steps = 2 * it.n;
            for (int x = 0; x < steps; ++x, ++rc) {
                const int hh = x / cnt, hx = x - hh * cnt;
                const int q_first = (i0 + (hx >> 1)) * BT + (hx & 1) * kDkvHalf;   // first query of the step
                const int h = it.h * r + hh;
                const int stage = rc % kDkvStages;
                if (lane == 0)
                    ok = mbar_wait(bar(kDkvBarRingEmpty + stage), ((rc / kDkvStages) & 1u) ^ 1u, abort_flag, 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = bar(kDkvBarRingFull + stage);
                    mbar_arrive_expect_tx(full, 2 * kHalfBytes);
                    const uint32_t dst = smem_base + kDkvSmemRing + stage * kDkvStageBytes;
#pragma unroll
                    for (int c = 0; c < kChunks; ++c) {
                        tma_load_4d(dst + c * kDkvHalfChunkBytes, &map_q, full, 64 * c, q_first, h, it.b);
                        tma_load_4d(dst + kDkvHalfTileBytes + c * kDkvHalfChunkBytes, &map_do, full, 64 * c, q_first, h, it.b);
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer: S^T, dP^T pairs ---------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_t = instr_desc_f16(BF16 ? 1 : 0, BT, kDkvHalf, false, false);
            constexpr uint32_t hi = desc_hi_sw128(1024);
            const uint32_t own_k = smem_base + kSmemOwn, own_v = own_k + kTileBytes;
            // D[128 keys x 64 queries] = own[keys x HD] * streamed[64 queries x HD]^T
            auto issue_t = [&](uint32_t d_col, uint32_t a_tile, uint32_t b_tile) {
                const uint32_t a0 = desc_lo_sw128(a_tile, 16), b0 = desc_lo_sw128(b_tile, 16);
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t sa = desc_step(c * kChunkBytes + i * 32);
                        const uint32_t sb = desc_step(c * kDkvHalfChunkBytes + i * 32);
                        if (c | i) mma_ss_lo<true>(tmem + d_col, a0 + sa, b0 + sb, hi, idesc_t);
                        else mma_ss_lo<false>(tmem + d_col, a0 + sa, b0 + sb, hi, idesc_t);
                    }
            };
            bool ok = true;
            uint32_t items = 0, rc = 0;   // items, steps so far
            Item it;
            for (int seq = 0; ok && get_item<true>(p, seq, &it); ++seq) {
                if (it.n <= 0) continue;
                const int steps = 2 * it.n;
                ok = mbar_wait(bar(kDkvBarOwnFull), items & 1u, abort_flag, 2);
                if (!ok) break;
                for (int x = 0; ok && x < steps; ++x) {
                    // S^T and dP^T of step c into buffer c & 1, once step c-2's P^T and dS^T have been consumed
                    const uint32_t c = rc + x, b = c & 1u;
                    ok = mbar_wait(bar(kDkvBarRingFull + c % kDkvStages), (c / kDkvStages) & 1u, abort_flag, 3);
                    if (!ok) break;
                    ok = mbar_wait(bar(kDkvBarBufFree + b), ((c >> 1) & 1u) ^ 1u, abort_flag, 7);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t ring = smem_base + kDkvSmemRing + (c % kDkvStages) * kDkvStageBytes;
                    issue_t(kColS + 64 * b, own_k, ring);
                    tc_commit(bar(kDkvBarSFull + b));
                    issue_t(kColDp + 64 * b, own_v, ring + kDkvHalfTileBytes);
                    tc_commit(bar(kDkvBarDpFull + b));
                }
                if (!ok) break;
                rc += steps;
                tc_commit(bar(kDkvBarOwnEmpty));
                ++items;
            }
        }
        __syncwarp();
    } else if (warp == kAccWarp) {
        // ------------------------------ MMA issuer: dV, dK -----------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_acc = instr_desc_f16(BF16 ? 1 : 0, BT, HD, false, true);
            constexpr uint32_t hi = desc_hi_sw128(1024);
            // D[128 keys x HD] (+)= A^T[keys x 64 queries] (16-bit, in TMEM) * streamed[64 queries x HD]
            auto issue_acc = [&](uint32_t d_col, uint32_t a_col, uint32_t b_tile, bool acc) {
                const uint32_t b0 = desc_lo_sw128(b_tile, kDkvHalfChunkBytes);
#pragma unroll
                for (int ks = 0; ks < kDkvHalf / 16; ++ks) {
                    // queries 0-31 sit in packed columns 0-15, queries 32-63 in columns 32-47: each
                    // half overlays the fp32 columns the warps that wrote it had read themselves
                    const uint32_t a = tmem + a_col + (ks < 2 ? ks * 8 : 32 + (ks - 2) * 8);
                    const uint32_t b = b0 + desc_step(ks * 16 * 128);
                    if (ks) mma_ts_lo<true>(tmem + d_col, a, b, hi, idesc_acc);
                    else mma_ts_lo(tmem + d_col, a, b, hi, idesc_acc, acc ? 1u : 0u);
                }
            };
            bool ok = true;
            uint32_t items = 0, rc = 0;
            Item it;
            for (int seq = 0; ok && get_item<true>(p, seq, &it); ++seq) {
                if (it.n <= 0) continue;
                const int steps = 2 * it.n;
                for (int x = 0; ok && x < steps; ++x) {
                    const uint32_t cur = rc + x, b = cur & 1u;
                    const uint32_t ring = smem_base + kDkvSmemRing + (cur % kDkvStages) * kDkvStageBytes;
                    ok = mbar_wait(bar(kDkvBarPFull), cur & 1u, abort_flag, 4);
                    if (!ok) break;
                    if (x == 0 && items > 0) {   // the previous item's dK / dV have been read out
                        ok = mbar_wait(bar(kDkvBarAccEmpty), (items - 1) & 1u, abort_flag, 5);
                        if (!ok) break;
                    }
                    tc_fence_after_sync();
                    issue_acc(kColDv, kColS + 64 * b, ring + kDkvHalfTileBytes, x > 0);   // dV += P^T dO
                    ok = mbar_wait(bar(kDkvBarDsFull), cur & 1u, abort_flag, 6);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_acc(kColDk, kColDp + 64 * b, ring, x > 0);                       // dK += dS^T Q
                    // (the pair issuer's reads of this stage finished before P^T could be formed)
                    tc_commit(bar(kDkvBarRingEmpty + cur % kDkvStages));
                    tc_commit(bar(kDkvBarBufFree + b));
                }
                if (!ok) break;
                rc += steps;
                tc_commit(bar(kDkvBarAccFull));
                ++items;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ element-wise warps -----------------------------------
        const int wg = warp >> 2, wq = warp & 3;
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        const int col0 = wg * 32;                        // this warp's query columns of the 64
        const float c2 = p.scale_log2;
        bool ok = true;
        uint32_t items = 0, rc = 0;
        Item it;
        for (int seq = 0; ok && get_item<true>(p, seq, &it); ++seq) {
            if (it.n < 0) continue;
            const int key = it.t * BT + wq * 32 + lane;
            const bool key_live = key < p.Lk;
            const int64_t out_row = (int64_t(it.b) * p.Hkv + it.h) * p.Lk + key;
            char* out = static_cast<char*>(wg == 0 ? p.dv : p.dk) + out_row * HD * 2;
            if (it.n == 0) {   // no query sees these keys: their gradients are zero
                if (key_live)
#pragma unroll
                    for (int v = 0; v < HD / 8; ++v) reinterpret_cast<uint4*>(out)[v] = make_uint4(0, 0, 0, 0);
                continue;
            }
            const int i0 = first_query_tile(p, it.t), cnt = 2 * (p.nq - i0);
            const int steps = 2 * it.n;
            int hh = 0, hx = 0;   // query head of the group and half tile within it (counted, not divided: this loop is the step)
            for (int x = 0; x < steps; ++x, ++rc) {
                const int q0 = (i0 + (hx >> 1)) * BT + (hx & 1) * kDkvHalf + col0;   // first query of this warp's columns
                const uint32_t b = rc & 1u;
                const uint32_t s_addr = tmem + lane_base + kColS + 64 * b + col0;
                const uint32_t dp_addr = tmem + lane_base + kColDp + 64 * b + col0;
                // The statistics of this warp's 32 queries, straight from the arrays the dQ kernel wrote (every
                // lane reads the same addresses: one transaction per load); issued before the wait for S^T.
                float4 st_lse[8], st_del[8];
                {
                    const int64_t prow = (int64_t(it.b) * p.Hq + it.h * r + hh) * (int64_t(p.nq) * BT) + q0;
                    const float4* gl = reinterpret_cast<const float4*>(p.nlse2 + prow);
                    const float4* gd = reinterpret_cast<const float4*>(p.nds + prow);
#pragma unroll
                    for (int v = 0; v < 8; ++v) { st_lse[v] = __ldg(gl + v); st_del[v] = __ldg(gd + v); }
                }
                if (++hx == cnt) { hx = 0; ++hh; }
                ok = mbar_wait(bar(kDkvBarSFull + b), (rc >> 1) & 1u, abort_flag, 11);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t s[32];
                tmem_ld32(s_addr, s);
                tmem_wait_ld();
                tmem_ld_fence32(s);
                // P^T[key, q] = exp2(S * c - lse2[q]); zero where the query does not see the key.
                // Two columns per instruction on the FMA pipe (fp32x2).
                const bool diag = p.causal && q0 < it.t * BT + BT;      // some query of these columns precedes some key
                const bool need_mask = diag || it.t * BT + BT > p.Lk;   // the same for the whole warp
                const float2 c22 = make_float2(c2, c2);
                uint32_t pk[16];
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const float4 l4 = st_lse[v];
                    const float2 e0 = ffma2(make_float2(__uint_as_float(s[4 * v]), __uint_as_float(s[4 * v + 1])), c22, make_float2(l4.x, l4.y));
                    const float2 e1 = ffma2(make_float2(__uint_as_float(s[4 * v + 2]), __uint_as_float(s[4 * v + 3])), c22, make_float2(l4.z, l4.w));
                    float pv[4] = {ex2_approx(e0.x), ex2_approx(e0.y), ex2_approx(e1.x), ex2_approx(e1.y)};
                    if (need_mask) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (!key_live || (diag && q0 + 4 * v + e < key)) pv[e] = 0.f;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[4 * v + e] = __float_as_uint(pv[e]);
                    pk[2 * v] = pack16<BF16>(pv[0], pv[1]);
                    pk[2 * v + 1] = pack16<BF16>(pv[2], pv[3]);
                }
                // 16-bit P^T over the first half of the fp32 columns this warp has just read
                tmem_st16(s_addr, pk);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kDkvBarPFull));
                // dS^T = P^T o (dP^T - delta[q]) * scale, with the unrounded P
                ok = mbar_wait(bar(kDkvBarDpFull + b), (rc >> 1) & 1u, abort_flag, 12);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t dp[32];
                tmem_ld32(dp_addr, dp);
                tmem_wait_ld();
                tmem_ld_fence32(dp);
                const float2 sc2 = make_float2(p.scale, p.scale);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const float4 d4 = st_del[v];   // -delta * scale
                    const float2 t0 = ffma2(make_float2(__uint_as_float(dp[4 * v]), __uint_as_float(dp[4 * v + 1])), sc2, make_float2(d4.x, d4.y));
                    const float2 t1 = ffma2(make_float2(__uint_as_float(dp[4 * v + 2]), __uint_as_float(dp[4 * v + 3])), sc2, make_float2(d4.z, d4.w));
                    const float2 d0 = fmul2(make_float2(__uint_as_float(s[4 * v]), __uint_as_float(s[4 * v + 1])), t0);
                    const float2 d1 = fmul2(make_float2(__uint_as_float(s[4 * v + 2]), __uint_as_float(s[4 * v + 3])), t1);
                    pk[2 * v] = pack16<BF16>(d0.x, d0.y);
                    pk[2 * v + 1] = pack16<BF16>(d1.x, d1.y);
                }
                tmem_st16(dp_addr, pk);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kDkvBarDsFull));
            }
            if (!ok) break;
            // read the item's accumulator out: warps 0-3 dV, warps 4-7 dK (one key row per lane)
            ok = mbar_wait(bar(kDkvBarAccFull), items & 1u, abort_flag, 13);
            if (!ok) break;
            ++items;
            tc_fence_after_sync();
            const uint32_t acc_addr = tmem + lane_base + (wg == 0 ? kColDv : kColDk);
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(acc_addr + 32 * c, o);
                tmem_wait_ld();
                tmem_ld_fence32(o);
                if (key_live) store_row32<BF16>(out + c * 64, o);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kDkvBarAccEmpty));
        }
    }

    // ------------------------------ common exit ------------------------------------------------
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

// ---------------------------------------------------------------------------------------------
// dQ: own pair = (Q_i, dO_i), streamed pair = (K_j, V_j).
// ---------------------------------------------------------------------------------------------
template <bool BF16, int HD>
__global__ void __launch_bounds__(kDkvThreads, 1)
sdpa_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto bar = [&](int i) { return smem_base + kDqSmemBars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kDqSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kDqSmemMisc + 4);
    constexpr int kChunks = HD / 64;
    constexpr uint32_t kLoadBytes = kChunks * kChunkBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = p.Hq / p.Hkv;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kDqNumBars; ++i) {
            const bool eight = i == kDqBarTaken || i == kDqBarDsFull || i == kDqBarAccEmpty;
            const bool two = i >= kDqBarStepFull && i < kDqBarStepFull + kDqFullBars;
            mbar_init(bar(i), eight ? 8u : (two ? 2u : 1u));
        }
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_base + kDqSmemMisc, kTmemCols);
        tmem_relinquish();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    constexpr int kColS = 0, kColDp = 128, kColDq = 256, kColDs = 384;   // dS: two buffers of 64 columns

    if (warp == kLoadWarp) {
        // ------------------------------ loads ------------------------------------------------
        if (lane == 0) {
            bool ok = true;
            uint32_t items = 0, rc = 0;
            Item it;
            for (int seq = 0; ok && get_item<false>(p, seq, &it); ++seq) {
                if (it.n <= 0) continue;
                const int hk = it.h / r;
                ok = mbar_wait(bar(kDqBarOwnEmpty), (items & 1u) ^ 1u, abort_flag, 0);
                if (!ok) break;
                ++items;
                mbar_arrive_expect_tx(bar(kDqBarOwnFull), 2 * kLoadBytes);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    tma_load_4d(smem_base + kSmemOwn + c * kChunkBytes, &map_q, bar(kDqBarOwnFull), 64 * c, it.t * BT, it.h, it.b);
                    tma_load_4d(smem_base + kSmemOwn + kTileBytes + c * kChunkBytes, &map_do, bar(kDqBarOwnFull), 64 * c, it.t * BT, it.h, it.b);
                }
                for (int x = 0; ok && x < it.n; ++x, ++rc) {
                    const uint32_t ks = rc % kDqKStages, vs = rc % kDqVStages;
                    ok = mbar_wait(bar(kDqBarKEmpty + ks), ((rc / kDqKStages) & 1u) ^ 1u, abort_flag, 1);
                    if (!ok) break;
                    const uint32_t full = bar(kDqBarStepFull + rc % kDqFullBars);
                    mbar_arrive_expect_tx(full, kLoadBytes);
#pragma unroll
                    for (int c = 0; c < kChunks; ++c)
                        tma_load_4d(smem_base + kDqSmemK + ks * kTileBytes + c * kChunkBytes, &map_k, full, 64 * c, x * BT, hk, it.b);
                    ok = mbar_wait(bar(kDqBarVEmpty + vs), ((rc / kDqVStages) & 1u) ^ 1u, abort_flag, 7);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full, kLoadBytes);
#pragma unroll
                    for (int c = 0; c < kChunks; ++c)
                        tma_load_4d(smem_base + kDqSmemV + vs * kTileBytes + c * kChunkBytes, &map_v, full, 64 * c, x * BT, hk, it.b);
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer -------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_kk = instr_desc_f16(BF16 ? 1 : 0, BT, BT, false, false);
            constexpr uint32_t idesc_acc = instr_desc_f16(BF16 ? 1 : 0, BT, HD, false, true);
            const uint32_t own_q = smem_base + kSmemOwn, own_do = own_q + kTileBytes;
            constexpr uint32_t hi = desc_hi_sw128(1024);
            // D[128 queries x 128 keys] = own[queries x HD] * streamed[keys x HD]^T
            auto issue_t = [&](uint32_t d_col, uint32_t a_tile, uint32_t b_tile) {
                const uint32_t a0 = desc_lo_sw128(a_tile, 16), b0 = desc_lo_sw128(b_tile, 16);
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t step = desc_step(c * kChunkBytes + i * 32);
                        if (c | i) mma_ss_lo<true>(tmem + d_col, a0 + step, b0 + step, hi, idesc_kk);
                        else mma_ss_lo<false>(tmem + d_col, a0 + step, b0 + step, hi, idesc_kk);
                    }
            };
            bool ok = true;
            uint32_t items = 0, rc = 0, pc = 0;
            Item it;
            for (int seq = 0; ok && get_item<false>(p, seq, &it); ++seq) {
                if (it.n <= 0) continue;
                auto k_tile = [&](uint32_t c) { return smem_base + kDqSmemK + (c % kDqKStages) * kTileBytes; };
                auto v_tile = [&](uint32_t c) { return smem_base + kDqSmemV + (c % kDqVStages) * kTileBytes; };
                // S = Q K^T and dP = dO V^T of step c; V's stage is free as soon as dP has run
                auto issue_s_dp = [&](uint32_t c) -> bool {
                    if (!mbar_wait(bar(kDqBarStepFull + c % kDqFullBars), (c / kDqFullBars) & 1u, abort_flag, 3)) return false;
                    tc_fence_after_sync();
                    issue_t(kColS, own_q, k_tile(c));
                    issue_t(kColDp, own_do, v_tile(c));
                    tc_commit(bar(kDqBarDpFull));   // covers S too: a commit tracks every MMA this thread has issued
                    tc_commit(bar(kDqBarVEmpty + c % kDqVStages));
                    return true;
                };
                ok = mbar_wait(bar(kDqBarOwnFull), items & 1u, abort_flag, 2);
                if (!ok) break;
                ok = issue_s_dp(rc);
                for (int x = 0; ok && x < it.n; ++x) {
                    // the element-wise warps hold S and dP of this step in registers: the next
                    // step's products (or the next item's first) may overwrite them while this
                    // step's dS is being formed
                    ok = mbar_wait(bar(kDqBarTaken), pc & 1u, abort_flag, 4);
                    if (!ok) break;
                    ++pc;
                    if (x + 1 < it.n) ok = issue_s_dp(rc + x + 1);
                }
                if (!ok) break;
                rc += it.n;
                tc_commit(bar(kDqBarOwnEmpty));   // every S / dP product of the item has read Q_i, dO_i
                ++items;
            }
        }
        __syncwarp();
    } else if (warp == kAccWarp) {
        // ------------------------------ second MMA issuer: dQ += dS K_j ------------------------
        // A thread of its own, so that its waits (dS formed, K landed) run while the first issuer is
        // blocked issuing S and dP of the next step, and the other way round.
        if (lane == 0) {
            constexpr uint32_t idesc_acc = instr_desc_f16(BF16 ? 1 : 0, BT, HD, false, true);
            constexpr uint32_t hi = desc_hi_sw128(1024);
            bool ok = true;
            uint32_t items = 0, rc = 0;
            Item it;
            for (int seq = 0; ok && get_item<false>(p, seq, &it); ++seq) {
                if (it.n <= 0) continue;
                for (int x = 0; ok && x < it.n; ++x) {
                    const uint32_t cur = rc + x;
                    ok = mbar_wait(bar(kDqBarDsFull), cur & 1u, abort_flag, 6);
                    if (!ok) break;
                    if (x == 0 && items > 0) {   // the previous item's dQ has been read out
                        ok = mbar_wait(bar(kDqBarAccEmpty), (items - 1) & 1u, abort_flag, 5);
                        if (!ok) break;
                    }
                    // K_j landed (the first issuer saw that before S; this thread reads the tile too)
                    ok = mbar_wait(bar(kDqBarStepFull + cur % kDqFullBars), (cur / kDqFullBars) & 1u, abort_flag, 9);
                    if (!ok) break;
                    tc_fence_after_sync();
                    // dS (16-bit) from TMEM, K_j as [keys x HD] rows
                    const uint32_t ds_col = kColDs + (cur & 1u) * 64;
                    const uint32_t k0 = desc_lo_sw128(smem_base + kDqSmemK + (cur % kDqKStages) * kTileBytes, kChunkBytes);
#pragma unroll
                    for (int ks = 0; ks < BT / 16; ++ks) {
                        if (ks) mma_ts_lo<true>(tmem + kColDq, tmem + ds_col + ks * 8, k0 + desc_step(ks * 16 * 128), hi, idesc_acc);
                        else mma_ts_lo(tmem + kColDq, tmem + ds_col, k0, hi, idesc_acc, x > 0 ? 1u : 0u);
                    }
                    tc_commit(bar(kDqBarKEmpty + cur % kDqKStages));
                    tc_commit(bar(kDqBarDsFree + (cur & 1u)));   // this dS buffer may be written again
                }
                if (!ok) break;
                rc += it.n;
                tc_commit(bar(kDqBarAccFull));
                ++items;
            }
        }
        __syncwarp();
    } else if (warp < 8) {
        // ------------------------------ element-wise warps -----------------------------------
        const int wg = warp >> 2, wq = warp & 3;
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        const int col0 = wg * 64;                        // this warp's key columns of the tile
        const uint32_t s_addr = tmem + lane_base + kColS + col0;
        const uint32_t dp_addr = tmem + lane_base + kColDp + col0;
        const float c2 = p.scale_log2;
        bool ok = true;
        uint32_t items = 0, rc = 0;
        Item it;
        for (int seq = 0; ok && get_item<false>(p, seq, &it); ++seq) {
            if (it.n <= 0) continue;
            const int row = it.t * BT + wq * 32 + lane;
            const bool live = row < p.Lq;
            const int64_t grow = (int64_t(it.b) * p.Hq + it.h) * p.Lq + row;
            // Row statistics.  delta = sum_d dO[row, d] * O[row, d] is formed here: the eight warps split
            // the tile's 128 rows sixteen each and read them as they lie in memory (a row is HD * 2
            // contiguous bytes, HD / 8 lanes per row), reduce within the lanes of a row and pass the sums
            // through shared memory to the threads that own the rows; the sums also go out for the
            // dK/dV kernel.  The item's S and dP are usually waiting by now, so this round trip is
            // exposed: the rows were asked into L2 when the previous item started.
            constexpr int LPR = HD / 8;        // lanes per row (16 bytes each)
            constexpr int RPI = 32 / LPR;      // rows per warp-wide load
            constexpr int NI = 16 / RPI;       // loads per tensor
            const int64_t tile_row0 = (int64_t(it.b) * p.Hq + it.h) * p.Lq + it.t * BT;
            const float nlse2 = live ? -p.lse[grow] * 1.4426950408889634f : -INFINITY;   // dead rows: P = exp2(-inf) = 0
            float delta;
            {
                float* xch = reinterpret_cast<float*>(smem_gen + kDqSmemDelta);
                uint4 ov[NI], dv[NI];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int rr = 16 * warp + i * RPI + lane / LPR;          // row within the tile
                    const bool valid = it.t * BT + rr < p.Lq;
                    const int64_t off = ((tile_row0 + rr) * HD) * 2 + (lane % LPR) * 16;
                    ov[i] = valid ? __ldg(reinterpret_cast<const uint4*>(static_cast<const char*>(p.out) + off)) : make_uint4(0, 0, 0, 0);
                    dv[i] = valid ? __ldg(reinterpret_cast<const uint4*>(static_cast<const char*>(p.dout) + off)) : make_uint4(0, 0, 0, 0);
                }
                {
                    // the next item's rows (16 per warp, both tensors) and statistics: towards L2
                    Item nx;
                    int sq = seq + 1;
                    bool have = get_item<false>(p, sq, &nx);
                    if (have && nx.n <= 0) have = get_item<false>(p, ++sq, &nx);
                    if (have && nx.n > 0) {
                        const int64_t nrow = (int64_t(nx.b) * p.Hq + nx.h) * p.Lq + nx.t * BT + 16 * warp;
                        if (nx.t * BT + 16 * warp < p.Lq) {
                            constexpr int kLines = 16 * HD * 2 / 128;       // 128-byte lines of 16 rows
                            if (lane < kLines) {
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(p.out) + nrow * HD * 2 + 128 * lane));
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(p.dout) + nrow * HD * 2 + 128 * lane));
                            }
                            if (lane == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.lse + nrow));
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const uint32_t ow[4] = {ov[i].x, ov[i].y, ov[i].z, ov[i].w};
                    const uint32_t dw[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 a = pair16_to_f32<BF16>(ow[e]), b = pair16_to_f32<BF16>(dw[e]);
                        part = fmaf(a.x, b.x, part);
                        part = fmaf(a.y, b.y, part);
                    }
#pragma unroll
                    for (int sh = LPR / 2; sh > 0; sh >>= 1) part += __shfl_xor_sync(0xffffffffu, part, sh);
                    if (lane % LPR == 0) xch[16 * warp + i * RPI + lane / LPR] = part;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight element-wise warps
                delta = xch[wq * 32 + lane];
                if (wg == 0) {   // every row of the tile, the ones past the end too
                    const int64_t prow = (int64_t(it.b) * p.Hq + it.h) * (int64_t(p.nq) * BT) + it.t * BT + wq * 32 + lane;
                    p.nds[prow] = live ? -delta * p.scale : 0.f;
                    p.nlse2[prow] = nlse2;
                }
            }
            for (int x = 0; x < it.n; ++x, ++rc) {
                // one wait for both products: dP is committed after S by the same thread
                ok = mbar_wait(bar(kDqBarDpFull), rc & 1u, abort_flag, 12);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t s[64], dp[64];
                tmem_ld32(s_addr, reinterpret_cast<uint32_t(&)[32]>(s[0]));
                tmem_ld32(s_addr + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
                tmem_ld32(dp_addr, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
                tmem_ld32(dp_addr + 32, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
                tmem_wait_ld();
                tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(s[0]));
                tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(s[32]));
                tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(dp[0]));
                tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(dp[32]));
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kDqBarTaken));   // S and dP are in registers
                // P = exp2(S * c - lse2), zero where the query does not see the key;
                // dS = P o (dP - delta) * scale
                const int k0 = x * BT + col0;
                const int limit = (p.causal ? min(row, p.Lk - 1) : p.Lk - 1) - k0;   // last visible column
                // some column of these 64 is invisible to some row of this warp (the same for all lanes)
                const bool need_mask = (p.causal && k0 + 63 > it.t * BT + wq * 32) || k0 + 64 > p.Lk;
                const float2 c22 = make_float2(c2, c2), nl2 = make_float2(nlse2, nlse2);
                const float2 sc2 = make_float2(p.scale, p.scale), nd2 = make_float2(-delta * p.scale, -delta * p.scale);
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float2 e = ffma2(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), c22, nl2);
                    float p0 = ex2_approx(e.x), p1 = ex2_approx(e.y);
                    if (need_mask) {
                        if (c > limit) p0 = 0.f;
                        if (c + 1 > limit) p1 = 0.f;
                    }
                    const float2 t = ffma2(make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), sc2, nd2);
                    const float2 d = fmul2(make_float2(p0, p1), t);
                    pk[c >> 1] = pack16<BF16>(d.x, d.y);
                }
                const uint32_t ds_addr = tmem + lane_base + kColDs + (rc & 1u) * 64 + wg * 32;
                // dQ of the step before last has consumed this buffer (its issuer runs on its own)
                ok = mbar_wait(bar(kDqBarDsFree + (rc & 1u)), ((rc >> 1) & 1u) ^ 1u, abort_flag, 14);
                if (!ok) break;
                tmem_st16(ds_addr, reinterpret_cast<uint32_t(&)[16]>(pk[0]));
                tmem_st16(ds_addr + 16, reinterpret_cast<uint32_t(&)[16]>(pk[16]));
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kDqBarDsFull));
            }
            if (!ok) break;
            ok = mbar_wait(bar(kDqBarAccFull), items & 1u, abort_flag, 13);
            if (!ok) break;
            ++items;
            tc_fence_after_sync();
            // warps 0-3 store the first half of the head dim, warps 4-7 the second
            const uint32_t acc_addr = tmem + lane_base + kColDq + wg * (HD / 2);
            char* out = static_cast<char*>(p.dq) + (grow * HD + wg * (HD / 2)) * 2;
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                uint32_t o[32];
                tmem_ld32(acc_addr + 32 * c, o);
                tmem_wait_ld();
                tmem_ld_fence32(o);
                if (live) store_row32<BF16>(out + c * 64, o);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kDqBarAccEmpty));
        }
    }

    // ------------------------------ common exit ------------------------------------------------
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

}  // namespace

bool sdpa_bwd_tc_supported(const Gpu* g, const paras_sdpa_bwd_args& a) {
    if (g->cc_major != 10) return false;
    if (a.dtype != PARAS_BF16 && a.dtype != PARAS_F16) return false;
    if (a.D != 128 && a.D != 64) return false;
    if (a.Lq < 1 || a.Lk < 1 || a.Hkv < 1 || a.Hq % a.Hkv) return false;
    if (!(a.scale > 0.0) || !std::isfinite(a.scale)) return false;
    if (g->smem_optin < size_t(kDkvSmemLaunch) || g->smem_optin < size_t(kDqSmemLaunch)) return false;
    return true;
}

// Scratch the two kernels share: the two per-query statistics arrays, rows padded to whole query tiles.
size_t sdpa_bwd_tc_scratch_bytes(const paras_sdpa_bwd_args& a) {
    const size_t rows = size_t(a.B) * a.Hq * size_t((a.Lq + BT - 1) / BT) * BT;
    return 2 * rows * sizeof(float);
}

// dq, dk, dv from dense [B, H, L, D] tensors; `scratch` has sdpa_bwd_tc_scratch_bytes(a) bytes.
int sdpa_bwd_tc_launch(Gpu* g, const paras_sdpa_bwd_args& a, float* scratch, cudaStream_t s) {
    int st = check_status_word(g);
    if (st != PARAS_OK) return st;
    const int64_t sq[3] = {int64_t(a.Hq) * a.Lq * a.D, int64_t(a.Lq) * a.D, a.D};
    const int64_t sk[3] = {int64_t(a.Hkv) * a.Lk * a.D, int64_t(a.Lk) * a.D, a.D};
    CUtensorMap mq, mk, mv, mdo;
    if ((st = make_tensor_map_bhld(&mq, a.q, a.dtype, a.B, a.Hq, a.Lq, a.D, sq, BT)) != PARAS_OK) return st;
    if ((st = make_tensor_map_bhld(&mk, a.k, a.dtype, a.B, a.Hkv, a.Lk, a.D, sk, BT)) != PARAS_OK) return st;
    if ((st = make_tensor_map_bhld(&mv, a.v, a.dtype, a.B, a.Hkv, a.Lk, a.D, sk, BT)) != PARAS_OK) return st;
    if ((st = make_tensor_map_bhld(&mdo, a.dout, a.dtype, a.B, a.Hq, a.Lq, a.D, sq, BT)) != PARAS_OK) return st;
    // the dK/dV kernel streams queries 64 rows at a time
    CUtensorMap mq64, mdo64;
    if ((st = make_tensor_map_bhld(&mq64, a.q, a.dtype, a.B, a.Hq, a.Lq, a.D, sq, kDkvHalf)) != PARAS_OK) return st;
    if ((st = make_tensor_map_bhld(&mdo64, a.dout, a.dtype, a.B, a.Hq, a.Lq, a.D, sq, kDkvHalf)) != PARAS_OK) return st;
    BwdParams p{};
    p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
    p.lse = a.lse; p.out = a.out; p.dout = a.dout;
    p.nlse2 = scratch;
    p.nds = scratch + size_t(a.B) * a.Hq * size_t((a.Lq + BT - 1) / BT) * BT;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk;
    p.causal = a.causal;
    p.scale = float(a.scale);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.status = g->status_dev;
    p.nq = (a.Lq + BT - 1) / BT;
    p.nk = (a.Lk + BT - 1) / BT;
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const bool bf = a.dtype == PARAS_BF16;
    const CUtensorMap* use_q = &mq;
    const CUtensorMap* use_do = &mdo;
    int threads = kDkvThreads;
    auto launch = [&](auto kernel, int64_t units, int smem) -> int {
        if (units > INT32_MAX) return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: too many work units");
        p.units = int(units);
        PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kernel<<<unsigned(units < sms ? units : sms), threads, smem, s>>>(*use_q, mk, mv, *use_do, p);
        return PARAS_OK;
    };
    // dQ: units of paired query tiles per (batch, query head); whole 128-row tiles of q and dO
    // (it also writes the per-query statistics the dK/dV kernel reads: this launch comes first)
    use_q = &mq;
    use_do = &mdo;
    p.npair = (p.nq + 1) / 2;
    const int64_t u_q = int64_t(a.B) * a.Hq * p.npair;
    if (a.D == 128) st = bf ? launch(sdpa_bwd_dq_kernel<true, 128>, u_q, kDqSmemLaunch) : launch(sdpa_bwd_dq_kernel<false, 128>, u_q, kDqSmemLaunch);
    else st = bf ? launch(sdpa_bwd_dq_kernel<true, 64>, u_q, kDqSmemLaunch) : launch(sdpa_bwd_dq_kernel<false, 64>, u_q, kDqSmemLaunch);
    if (st != PARAS_OK) return st;
    PB_LAUNCH_CHECK("sdpa_bwd_dq_kernel");
    // dK, dV: units of paired key tiles per (batch, kv head); queries stream 64 rows at a time
    use_q = &mq64;
    use_do = &mdo64;
    threads = kDkvThreads;
    p.npair = (p.nk + 1) / 2;
    const int64_t u_kv = int64_t(a.B) * a.Hkv * p.npair;
    if (a.D == 128) st = bf ? launch(sdpa_bwd_dkv_kernel<true, 128>, u_kv, kDkvSmemLaunch) : launch(sdpa_bwd_dkv_kernel<false, 128>, u_kv, kDkvSmemLaunch);
    else st = bf ? launch(sdpa_bwd_dkv_kernel<true, 64>, u_kv, kDkvSmemLaunch) : launch(sdpa_bwd_dkv_kernel<false, 64>, u_kv, kDkvSmemLaunch);
    if (st != PARAS_OK) return st;
    PB_LAUNCH_CHECK("sdpa_bwd_dkv_kernel");
    return PARAS_OK;
}

}  // namespace pb
