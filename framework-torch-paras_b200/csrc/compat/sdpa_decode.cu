// Split-KV attention for short queries over a long K/V cache (the decode step): HBM-bound.
//
// Reference path being replaced for this shape: sdpa_math with enable_gqa
// (csrc/ops/attention_ops.cpp:83-93) first expands K and V from Hkv to Hq heads
// (repeat_interleave, csrc/ops/tensor_ops.cpp:687-729: 2.1 GB -> 8.6 GB per tensor at
// B=64, kv_len=32768), then runs the composition.  Here every K/V byte is read from HBM
// exactly once: the (Hq/Hkv) query heads that share a kv head, times the few query
// positions, form the <= 16 rows of one m16n8k16 tensor-core tile, so one pass over the
// kv head's cache serves all of them.  Algorithmic traffic = K + V (once per kv head) + q + o.
//
// One CTA = one (batch, kv head, key range).  A producer warp streams 64-key K and V tiles
// through a 6-stage shared-memory ring with TMA (128-byte swizzle, 192 KB in flight per SM);
// four consumer warps each take 16 keys of a tile: S = Q K^T with mma.sync (fp32
// accumulate), online softmax in registers, O += P V with the P fragments reused straight
// from the S accumulators.  The four warps' (max, sum, O) states are merged through shared
// memory at the end; with more than one key range per kv head the CTA writes an fp32
// partial and sdpa_combine_kernel merges the ranges.
//
// The tensor-core rate needed is small (16 FLOP per K/V byte with 4x row padding), so the
// legacy mma.sync path is ample; tcgen05 with its 128-row tiles would waste 32x instead.
#include <algorithm>
#include <cmath>

#include "sdpa_common.cuh"
#include "tc_prims.cuh"
#include "tma_host.cuh"

namespace pb {
namespace {

using namespace tc;

constexpr int TK = 64;                       // keys per tile
constexpr int kStages = 6;
constexpr int kHalfBytes = 64 * 2 * TK;      // one 64-wide half of the head dim: 64 keys x 128 B
constexpr int kTileBytes = 2 * kHalfBytes;   // 16 KB (K or V tile)
constexpr int kStageBytes = 2 * kTileBytes;  // K tile + V tile
constexpr int kConsumers = 4;
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kSmemBars = kStages * kStageBytes;
constexpr int kSmemMisc = kSmemBars + 2 * kStages * 8;
constexpr int kSmemLaunch = kSmemMisc + 16 + 1024;
constexpr int kMaxRows = 16;

struct DecParams {
    const void* q;
    void* out;
    float* lse;
    int B, Hq, Hkv, Lq, Lk, group, rows;  // rows = group * Lq <= 16
    int64_t qs[3], os[3];
    int causal;
    float scale, scale_log2;
    int splits, tiles_per_split;
    float* o_part;
    float2* ml_part;
    int* status;
    // explicit attn_mask [B, Hq, Lq, Lk] (element strides, 0 = broadcast): 1 bool, 2 additive in the
    // tensors' dtype, 3 additive fp32; additive values join the unscaled scores divided by the scale
    const void* mask;
    int mask_kind;
    int64_t ms[4];
    float inv_scale;
    float masked_below;   // an additive mask entry at or below this removes its key (-inf, or -60000 when the scale allows)
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// Byte offset of (row, 16-byte chunk `c16` of the 128-byte line) inside a TMA 128B-swizzled
// half tile whose base is 1024-byte aligned.
__device__ __forceinline__ uint32_t swz(int row, int c16) {
    return uint32_t(row * 128 + ((c16 ^ (row & 7)) << 4));
}

// HD = 128, or 64: the same tile layout with only the first 64-wide half of every K / V tile loaded and used.
template <bool BF16, bool MASK, int HD>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const DecParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto full = [&](int s) { return smem_base + kSmemBars + 8u * s; };
    auto empty = [&](int s) { return smem_base + kSmemBars + 8u * (kStages + s); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kSmemMisc);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    int total_tiles = (p.Lk + TK - 1) / TK;
    int tiles_per_split = p.tiles_per_split;
    int* last_valid = reinterpret_cast<int*>(smem_gen + kSmemMisc + 4);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), kConsumers);
        }
        *abort_flag = 0;
        *last_valid = -1;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    // A mask that is one row of keys per batch element (caches of different lengths, padded to a common
    // length), bool or additive with entries 0 / -inf: the keys after the last one that may be attended are
    // never loaded.  The CTAs of a batch element find that key (a pass over the mask row) and share the shorter
    // range out among themselves; when the valid keys form a prefix the mask is not read again at all.
    // An additive row with any other value is a bias, not a padding mask, and is applied as given.
    int last_key = p.Lk - 1;      // the last key that may be attended
    bool mask_off = false;        // the key range says everything the mask says
    if (MASK && p.ms[1] == 0 && p.ms[2] == 0 && p.ms[3] == 1) {
        int* s_count = last_valid + 1;
        int* s_other = last_valid + 2;
        if (threadIdx.x == 0) { *s_count = 0; *s_other = 0; }
        __syncthreads();
        const int esz = p.mask_kind == 1 ? 1 : p.mask_kind == 2 ? 2 : 4;
        const unsigned char* row = static_cast<const unsigned char*>(p.mask) + int64_t(b) * p.ms[0] * esz;
        int last = -1, count = 0;
        bool other = false;
        auto take = [&](int k, bool valid, bool masked) {
            if (valid) { last = k; ++count; }
            else if (!masked) other = true;
        };
        if (p.mask_kind == 1 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0 && p.Lk % 16 == 0) {
            for (int c = int(threadIdx.x); c < p.Lk / 16; c += kThreads) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(row) + c);
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) take(16 * c + 4 * j + e, ((ww[j] >> (8 * e)) & 0xffu) != 0, true);
            }
        } else {
            for (int k = int(threadIdx.x); k < p.Lk; k += kThreads) {
                if (p.mask_kind == 1) {
                    take(k, row[k] != 0, true);
                } else {
                    const float f = p.mask_kind == 2 ? from16<BF16>(__ldg(reinterpret_cast<const uint16_t*>(row) + k))
                                                     : __ldg(reinterpret_cast<const float*>(row) + k);
                    take(k, f == 0.f, f <= p.masked_below);
                }
            }
        }
        if (last >= 0) atomicMax(last_valid, last);
        if (count) atomicAdd(s_count, count);
        if (other) atomicOr(s_other, 1);
        __syncthreads();
        if (*s_other == 0 && *last_valid >= 0) {
            last_key = *last_valid;
            mask_off = *s_count == last_key + 1;
            total_tiles = (last_key + 1 + TK - 1) / TK;
            tiles_per_split = (total_tiles + int(gridDim.x) - 1) / int(gridDim.x);
        }
    }
    const int t0 = split * tiles_per_split;
    const int t1 = min(total_tiles, t0 + tiles_per_split);
    const int ntiles = max(0, t1 - t0);

    // per-thread softmax state for rows r0 = lane/4 and r0 + 8, and the O accumulators
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc_o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_o[i][e] = 0.f;

    if (warp == kConsumers) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            for (int i = 0; i < ntiles; ++i) {
                const int s = i % kStages;
                if (!mbar_wait(empty(s), ((i / kStages) & 1) ^ 1u, abort_flag)) break;
                mbar_arrive_expect_tx(full(s), 2 * (HD / 64) * kHalfBytes);
                const uint32_t dst = smem_base + s * kStageBytes;
                const int key0 = (t0 + i) * TK;
                tma_load_4d(dst, &map_k, full(s), 0, key0, hk, b);
                if (HD > 64) tma_load_4d(dst + kHalfBytes, &map_k, full(s), 64, key0, hk, b);
                tma_load_4d(dst + kTileBytes, &map_v, full(s), 0, key0, hk, b);
                if (HD > 64) tma_load_4d(dst + kTileBytes + kHalfBytes, &map_v, full(s), 64, key0, hk, b);
            }
        }
    } else {
        // ------------------------------ consumers ----------------------------------
        // Row r of the 16-row tile = query position r / group of query head hk*group + r % group.
        const int r0 = lane >> 2, cpair = (lane & 3) * 2;
        uint32_t qf[HD / 16][4];
        {
            const uint16_t* qbase = static_cast<const uint16_t*>(p.q);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = r0 + 8 * half;
                const bool live = r < p.rows;
                const int qi = live ? r / p.group : 0, hh = live ? r % p.group : 0;
                const uint16_t* qrow = qbase + int64_t(b) * p.qs[0] + int64_t(hk * p.group + hh) * p.qs[1] +
                                       int64_t(qi) * p.qs[2];
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    // a0/a1: d = ks*16 + cpair (+1); a2/a3: d + 8
                    qf[ks][half] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + cpair) : 0u;
                    qf[ks][2 + half] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + cpair) : 0u;
                }
            }
        }
        const float c2 = p.scale_log2;
        int lim[2];  // last key each of this thread's two rows may attend
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = r0 + 8 * half;
            lim[half] = last_key;
            if (p.causal && r < p.rows) lim[half] = min(lim[half], r / p.group);  // top-left aligned
        }
        int64_t mrow[2] = {0, 0};   // element offset of each row's mask entries for key 0
        if (MASK) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = min(r0 + 8 * half, p.rows - 1);
                mrow[half] = int64_t(b) * p.ms[0] + int64_t(hk * p.group + r % p.group) * p.ms[1] + int64_t(r / p.group) * p.ms[2];
            }
        }
        // A bool mask with contiguous keys whose two rows share a mask row (a key-padding mask): this thread's
        // four bytes of a tile are two aligned 2-byte loads, asked for a tile ahead so that their latency runs
        // under the tile before (after the MMAs, where the mask is needed, nothing else could hide it).
        const bool mfast = MASK && p.mask_kind == 1 && p.ms[3] == 1 && mrow[0] == mrow[1] &&
                           ((reinterpret_cast<uintptr_t>(p.mask) + size_t(mrow[0])) & 1u) == 0;
        auto mask_pair = [&](int i) -> uint32_t {   // keys +0, +1 in the low half, +8, +9 in the high half
            const int kb = (t0 + i) * TK + warp * 16 + cpair;
            if (i >= ntiles || kb + 9 >= p.Lk) return 0u;
            const unsigned char* mp = static_cast<const unsigned char*>(p.mask) + mrow[0] + kb;
            return uint32_t(__ldg(reinterpret_cast<const uint16_t*>(mp))) | (uint32_t(__ldg(reinterpret_cast<const uint16_t*>(mp + 8))) << 16);
        };
        uint32_t mnext = mfast && !mask_off ? mask_pair(0) : 0u;
        bool ok = true;
        for (int i = 0; i < ntiles; ++i) {
            const int s = i % kStages;
            const int krow0 = warp * 16;  // this warp's 16 keys inside the tile
            const int key_base = (t0 + i) * TK + krow0 + cpair;
            const uint32_t mcur = mnext;
            if (mfast && !mask_off) mnext = mask_pair(i + 1);
            ok = mbar_wait(full(s), (i / kStages) & 1, abort_flag);
            if (!ok) break;
            const uint32_t kbase = smem_base + s * kStageBytes;
            const uint32_t vbase = kbase + kTileBytes;

            // ---- S = Q K^T for 16 keys: two n-tiles of 8 keys ----
            float acc_s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks2 = 0; ks2 < HD / 32; ++ks2) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    // four 8x8 blocks: keys nt*8..+7, d = ks2*32 + {0,8,16,24}
                    const int row = krow0 + nt * 8 + (lane & 7);
                    const int d0 = ks2 * 32 + (lane >> 3) * 8;
                    uint32_t bf[4];
                    ldmatrix_x4(kbase + (d0 >> 6) * kHalfBytes + swz(row, (d0 & 63) >> 3), bf);
                    mma16816<BF16>(acc_s[nt], qf[2 * ks2], bf[0], bf[1]);
                    mma16816<BF16>(acc_s[nt], qf[2 * ks2 + 1], bf[2], bf[3]);
                }
            }
            // ---- mask, online softmax ----
            // what the mask adds to this thread's four keys of each of its two rows (one set of loads when the
            // rows share a mask row, as with a key-padding mask)
            float madd[2][2][2];
            if (MASK && mask_off) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) madd[0][nt][e] = madd[1][nt][e] = 0.f;
            } else if (MASK && mfast && key_base + 9 < p.Lk) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        madd[0][nt][e] = madd[1][nt][e] = ((mcur >> (16 * nt + 8 * e)) & 0xffu) ? 0.f : -INFINITY;
            } else if (MASK) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half == 1 && mrow[1] == mrow[0]) {
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                            for (int e = 0; e < 2; ++e) madd[1][nt][e] = madd[0][nt][e];
                        continue;
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int key = min(key_base + nt * 8 + e, p.Lk - 1);
                            const int64_t mo = mrow[half] + int64_t(key) * p.ms[3];
                            float a;
                            if (p.mask_kind == 1) a = __ldg(static_cast<const unsigned char*>(p.mask) + mo) ? 0.f : -INFINITY;
                            else if (p.mask_kind == 2) a = from16<BF16>(__ldg(static_cast<const uint16_t*>(p.mask) + mo)) * p.inv_scale;
                            else a = __ldg(static_cast<const float*>(p.mask) + mo) * p.inv_scale;
                            madd[half][nt][e] = a;
                        }
                }
            }
            float p_[2][4];
            float alpha[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float mx = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key_base + nt * 8 + e;
                        float v = acc_s[nt][2 * half + e];
                        if (key > lim[half]) v = -INFINITY;
                        else if (MASK) v += madd[half][nt][e];   // -inf for a masked-out key
                        acc_s[nt][2 * half + e] = v;
                        mx = fmaxf(mx, v);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[half], mx);
                float sum = 0.f;
                if (m_new == -INFINITY) {
                    alpha[half] = 1.f;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) p_[nt][2 * half + e] = 0.f;
                } else {
                    alpha[half] = ex2_approx((m_run[half] - m_new) * c2);
                    const float neg = -m_new * c2;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float pv = ex2_approx(fmaf(acc_s[nt][2 * half + e], c2, neg));
                            p_[nt][2 * half + e] = pv;
                            sum += pv;
                        }
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                l_run[half] = l_run[half] * alpha[half] + sum;
                m_run[half] = m_new;
            }
#pragma unroll
            for (int i2 = 0; i2 < HD / 8; ++i2) {
                acc_o[i2][0] *= alpha[0];
                acc_o[i2][1] *= alpha[0];
                acc_o[i2][2] *= alpha[1];
                acc_o[i2][3] *= alpha[1];
            }
            // ---- O += P V : P (16 rows x 16 keys) straight from the S accumulators ----
            uint32_t pa[4];
            pa[0] = pack16<BF16>(p_[0][0], p_[0][1]);
            pa[1] = pack16<BF16>(p_[0][2], p_[0][3]);
            pa[2] = pack16<BF16>(p_[1][0], p_[1][1]);
            pa[3] = pack16<BF16>(p_[1][2], p_[1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                // transposed 8x8 blocks: (keys 0-7 | 8-15) x (d = n2*16 + {0, 8})
                const int row = krow0 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int d0 = n2 * 16 + (lane >> 4) * 8;
                uint32_t bf[4];
                ldmatrix_x4_trans(vbase + (d0 >> 6) * kHalfBytes + swz(row, (d0 & 63) >> 3), bf);
                mma16816<BF16>(acc_o[2 * n2], pa, bf[0], bf[1]);
                mma16816<BF16>(acc_o[2 * n2 + 1], pa, bf[2], bf[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));
        }
    }

    // ---- merge the four warps through shared memory (the ring is drained by now) ----
    __syncthreads();
    float* m_sm = reinterpret_cast<float*>(smem_gen);                 // [4][16]
    float* l_sm = m_sm + kConsumers * kMaxRows;                        // [4][16]
    float* o_sm = l_sm + kConsumers * kMaxRows;                        // [4][rows<=16][128]
    if (warp < kConsumers) {
        const int r0 = lane >> 2, cpair = (lane & 3) * 2;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = r0 + 8 * half;
            if ((lane & 3) == 0) {
                m_sm[warp * kMaxRows + r] = m_run[half];
                l_sm[warp * kMaxRows + r] = l_run[half];
            }
            if (r < p.rows) {
#pragma unroll
                for (int i2 = 0; i2 < HD / 8; ++i2) {
                    float* dst = o_sm + (warp * kMaxRows + r) * HD + i2 * 8 + cpair;
                    dst[0] = acc_o[i2][2 * half];
                    dst[1] = acc_o[i2][2 * half + 1];
                }
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < p.rows * HD; idx += kThreads) {
        const int r = idx / HD, d = idx - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumers; ++w) m = fmaxf(m, m_sm[w * kMaxRows + r]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumers; ++w) {
            const float mw = m_sm[w * kMaxRows + r];
            if (mw != -INFINITY) {
                const float f = ex2_approx((mw - m) * p.scale_log2);
                l = fmaf(l_sm[w * kMaxRows + r], f, l);
                o = fmaf(o_sm[(w * kMaxRows + r) * HD + d], f, o);
            }
        }
        const int qi = r / p.group, h = hk * p.group + r % p.group;
        const int64_t row = (int64_t(b) * p.Hq + h) * p.Lq + qi;
        if (p.splits > 1) {
            const int64_t rows_total = int64_t(p.B) * p.Hq * p.Lq;
            p.o_part[(int64_t(split) * rows_total + row) * HD + d] = o;
            // partial max is kept in natural-log units of the scaled scores, as the combine kernel expects
            if (d == 0) p.ml_part[int64_t(split) * rows_total + row] = make_float2(m * p.scale, l);
        } else {
            uint16_t* orow = static_cast<uint16_t*>(p.out) + int64_t(b) * p.os[0] + int64_t(h) * p.os[1] +
                             int64_t(qi) * p.os[2];
            const float val = (l == 0.f) ? __int_as_float(0x7fc00000) : o / l;
            if constexpr (BF16) orow[d] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
            else orow[d] = __half_as_ushort(__float2half_rn(val));
            if (p.lse && d == 0) p.lse[row] = (l == 0.f) ? -INFINITY : m * p.scale + logf(l);
        }
    }
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = 2;
        __threadfence_system();
    }
}

int make_kv_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int L, int D, const int64_t* st) {
    return make_tensor_map_bhld(map, base, dtype, B, H, L, D, st, TK);
}

bool kv_strides_ok(const void* base, const int64_t* st, int B, int H, int L, int D) {
    if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
    if (L > 1 && (st[2] < D || (st[2] * 2) % 16)) return false;
    if (H > 1 && (st[1] <= 0 || (st[1] * 2) % 16)) return false;
    if (B > 1 && (st[0] <= 0 || (st[0] * 2) % 16)) return false;
    return true;
}

}  // namespace

bool sdpa_decode_supported(const Gpu* g, const paras_sdpa_args& a, const char** why) {
    *why = "";
    if (g->cc_major < 9) { *why = "GPU has no TMA"; return false; }
    if (a.dtype != PARAS_BF16 && a.dtype != PARAS_F16) { *why = "dtype is not 16-bit"; return false; }
    if (a.D != 128 && a.D != 64) { *why = "head dim is neither 128 nor 64"; return false; }
    if (a.mask && (a.mask_kind < 1 || a.mask_kind > 3)) { *why = "unknown mask kind"; return false; }
    if (a.Hkv < 1 || a.Lq < 1 || int64_t(a.Lq) * (a.Hq / a.Hkv) > kMaxRows) {
        *why = "more than 16 query rows per kv head";
        return false;
    }
    if (a.Lk < 512) { *why = "cache too short to be worth a streaming kernel"; return false; }
    if (!(a.scale > 0.0) || !std::isfinite(a.scale)) { *why = "scale is not positive"; return false; }
    if (a.Hkv > 65535 || a.B > 65535) { *why = "batch or heads exceed the grid limit"; return false; }
    if (g->smem_optin < size_t(kSmemLaunch)) { *why = "not enough shared memory"; return false; }
    if (!kv_strides_ok(a.k, a.k_strides, a.B, a.Hkv, a.Lk, a.D) || !kv_strides_ok(a.v, a.v_strides, a.B, a.Hkv, a.Lk, a.D)) {
        *why = "K/V pointers or strides are not 16-byte aligned";
        return false;
    }
    if ((reinterpret_cast<uintptr_t>(a.q) & 3u) || (a.q_strides[0] & 1) || (a.q_strides[1] & 1) || (a.q_strides[2] & 1)) {
        *why = "q is not 4-byte aligned";
        return false;
    }
    return true;
}

// Key ranges per kv head: enough CTAs to fill the GPU, as few partial waves as possible
// (one CTA per SM is resident: the ring takes 192 KB of shared memory).
int sdpa_decode_pick_splits(const Gpu* g, const paras_sdpa_args& a) {
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const int64_t units = int64_t(a.B) * a.Hkv;
    const int tiles = (a.Lk + TK - 1) / TK;
    const int max_splits = std::max(1, std::min(64, tiles / 8));
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= max_splits; ++s) {
        const double w = double(units) * s;
        const double waves = std::ceil(w / sms);
        // time ~ waves * (tiles per CTA + fixed per-CTA overhead of ~6 tiles)
        const double cost = waves * (double((tiles + s - 1) / s) + 6.0);
        if (cost < best_cost * 0.995) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

int sdpa_decode_launch(Gpu* g, const paras_sdpa_args& a, float scale, const SplitWorkspace& ws,
                       cudaStream_t s) {
    int st = check_status_word(g);
    if (st != PARAS_OK) return st;
    CUtensorMap mk, mv;
    if ((st = make_kv_map(&mk, a.k, a.dtype, a.B, a.Hkv, a.Lk, a.D, a.k_strides)) != PARAS_OK) return st;
    if ((st = make_kv_map(&mv, a.v, a.dtype, a.B, a.Hkv, a.Lk, a.D, a.v_strides)) != PARAS_OK) return st;
    DecParams p{};
    p.q = a.q; p.out = a.out; p.lse = a.lse;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk;
    p.group = a.Hq / a.Hkv;
    p.rows = p.group * a.Lq;
    for (int i = 0; i < 3; ++i) { p.qs[i] = a.q_strides[i]; p.os[i] = a.o_strides[i]; }
    p.causal = a.causal;
    p.scale = scale;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.splits = ws.splits;
    const int tiles = (a.Lk + TK - 1) / TK;
    p.tiles_per_split = (tiles + ws.splits - 1) / ws.splits;
    p.o_part = ws.o_part;
    p.ml_part = ws.ml_part;
    p.status = g->status_dev;
    p.mask = a.mask;
    p.mask_kind = a.mask ? a.mask_kind : 0;
    for (int i = 0; i < 4; ++i) p.ms[i] = a.mask_strides[i];
    // a dimension of extent 1 is never stepped along: its stride reads as 0, like a broadcast one
    if (a.B == 1) p.ms[0] = 0;
    if (a.Hq == 1) p.ms[1] = 0;
    if (a.Lq == 1) p.ms[2] = 0;
    if (a.Lk == 1) p.ms[3] = 1;
    p.inv_scale = 1.0f / scale;
    // -60000 (fp16's most negative values) times scale * log2(e) must be far below the -149 at which exp2 gives 0
    p.masked_below = scale * 1.4426950408889634f * 60000.0f > 1000.0f ? -60000.0f : -INFINITY;
    dim3 grid(ws.splits, a.Hkv, a.B);
    auto go = [&](auto kernel) -> int {
        PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLaunch));
        kernel<<<grid, kThreads, kSmemLaunch, s>>>(mk, mv, p);
        return PARAS_OK;
    };
    if (a.D == 128) {
        if (a.dtype == PARAS_BF16) st = a.mask ? go(sdpa_decode_kernel<true, true, 128>) : go(sdpa_decode_kernel<true, false, 128>);
        else st = a.mask ? go(sdpa_decode_kernel<false, true, 128>) : go(sdpa_decode_kernel<false, false, 128>);
    } else {
        if (a.dtype == PARAS_BF16) st = a.mask ? go(sdpa_decode_kernel<true, true, 64>) : go(sdpa_decode_kernel<true, false, 64>);
        else st = a.mask ? go(sdpa_decode_kernel<false, true, 64>) : go(sdpa_decode_kernel<false, false, 64>);
    }
    if (st != PARAS_OK) return st;
    PB_LAUNCH_CHECK("sdpa_decode_kernel");
    if (ws.splits > 1) return sdpa_combine_launch(g, a, ws, s);
    return PARAS_OK;
}

}  // namespace pb
