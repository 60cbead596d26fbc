// Flash attention forward for sm_100a: tcgen05 tensor cores, TMEM accumulators, TMA-fed
// K/V ring, warp-specialised roles.  16-bit tensors, head dim 128 or 64, causal (top-left
// aligned, csrc/ops/attention_ops.cpp:103-116), full, or explicitly masked (bool / additive,
// attention_ops.cpp:117-126) attention, GQA by indexing the
// shared kv head (never materialising the repeat_interleave of attention_ops.cpp:83-93).
//
// One CTA owns 256 consecutive query rows of one (batch, head) as two 128-row tiles that
// ping-pong: while the tensor core runs tile 0's MMAs, tile 1's softmax runs on the CUDA
// cores, and vice versa.
//
//   warps 0-3   softmax of query tile 0: one thread per row (TMEM lane = row)
//   warps 4-7   softmax of query tile 1
//   warp  8     allocates TMEM, then one lane issues every tcgen05.mma
//   warp  9     one lane issues every TMA load
//   warps 10-11 idle: they complete the third warpgroup, so that setmaxnreg can move their
//               registers (and most of warps 8-9's) to the softmax warps, which hold a whole
//               128-column S row per thread
//
// TMEM (512 columns x 128 lanes, fp32): S0 @0, S1 @128, O0 @256, O1 @384.  The 16-bit
// probabilities P_t overwrite the first 64 columns of S_t and feed the P*V MMA straight
// from TMEM.  Shared memory, all 128-byte swizzled as TMA writes it: Q 2x32 KB; a K/V ring
// of 2x64 KB whose slots hold the pair (V_j, K_j+1) that one step of the MMA loop consumes
// -- the single issuing thread is the busiest resource of the CTA (an mbarrier wait costs it
// about 200 cycles even when the barrier has long completed), so it gets one full wait and
// one release commit per step instead of one per tile; and 8x4 KB (one per softmax warp)
// through which finished O rows leave as TMA stores: a lane owns a row, so direct global
// stores would be 32 cache lines per instruction and hold up the load/store path the TMEM
// traffic shares.
//
// Per kv tile j and query tile t:  S_t = Q_t K_j^T  (8 MMAs, K=16 each)
//                                  P_t = exp2(S_t*c - m_t*c), row sums l_t
//                                  O_t += P_t V_j     (8 MMAs)
// m_t is a per-row reference, not the running max: it is the row max of the item's first kv
// tile, and afterwards only moves (with O_t and l_t rescaled in TMEM) when a tile's row sum
// shows that it has fallen behind by more than 2^8.  Any reference gives the exact O/l as long
// as P, l and O use it consistently; not looking for each tile's max first takes a full pass
// over the row off the chain  S ready -> P ready -> next S  that bounds the kernel.  A tile
// whose sums say that P may overflow is redone against its true max before P is stored.
//
// Instantiations beside the plain and the masked kernel (each pays only for what it uses; an index added to the
// softmax chain at run time costs the plain kernel 2-3 %):
//   ROPE   the query tile is rotated in shared memory before its first MMA (rotary embedding)
//   SPLIT  few query blocks against a long key range: units take pieces of the key range, sdpa_tc_combine_kernel
//          merges the partial outputs by their log-sum-exp
//   PACK   the query heads of a GQA group share an item when group x Lq <= 256 (rows = (head, position))
//   LENS   a key count per batch element (what a key-padding mask, or the causal mask over right-padded
//          sequences, turns into after key_mask_scan_kernel / causal_check_kernel have looked at it)
// and a gate (TcParams::gate) by which one of two launches made for the same call returns at once: the device,
// not the host, knows what the mask check found.
//
// Every wait is bounded (tc_prims.cuh); a wait that runs out raises the CTA's abort flag,
// all roles fall through to the common exit, TMEM is freed and the GPU's status word is set to
// a mask of the waits that were pending (bits: 0-1 Q buffer free, 2 ring slot free, 3 K/V
// landed, 4-5 Q landed, 6-7 P ready, 10-11 S ready, 16-17 last PV done).
#include <cmath>

#include "sdpa_common.cuh"
#include "tc_prims.cuh"
#include "tma_host.cuh"

namespace pb {
namespace {

using namespace tc;

constexpr int BM = 128;            // query rows per tile (MMA M)
constexpr int BN = 128;            // keys per tile (MMA N of QK^T, K of PV)
constexpr int kMaxHD = 128;        // head dim: 128 or 64 (template parameter HD); shared memory and TMEM are laid out for 128
constexpr int kTilesPerCta = 2;
constexpr int kStages = 2;         // K/V ring slots; a slot holds the pair (V_j, K_j+1) that one step consumes
constexpr int kChunkBytes = 64 * 2 * 128;    // 64 elements x 128 rows
constexpr int kTileBytes = 2 * kChunkBytes;  // 128 x 128 x 2 B
constexpr int kSoftmaxWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 9;
constexpr int kThreads = 384;       // warps 10-11 only complete the third warpgroup (setmaxnreg works on warpgroups)
// Registers per thread after setmaxnreg.  A scheduler hosts two softmax warps and one of warps
// 8-11: 2*200 + 96 = 496 of its 512 registers per lane.  setmaxnreg.inc waits (without a bound)
// until the registers it asks for are free, so the sum must stay below the file's size with
// room to spare: a split that fitted exactly never got past the instruction.
constexpr int kRegsSoftmax = 200, kRegsIssue = 96;
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;  // + 128 * tile
constexpr float kRescaleSum = 256.0f;         // a tile's row sum above this moves the reference
constexpr float kRedoSum = 32768.0f;          // a tile's row sum above this (every P is below it) redoes the tile

constexpr int kSmemQ = 0;
constexpr int kSmemKV = kTilesPerCta * kTileBytes;
constexpr int kPairBytes = 2 * kTileBytes;   // V tile, then K tile
constexpr int kSmemO = kSmemKV + kStages * kPairBytes;   // per softmax warp: 32 rows x 128 B staging for the O store
constexpr int kOStageBytes = 32 * 128;
constexpr int kSmemBars = kSmemO + kSoftmaxWarps * kOStageBytes;
// barrier indices
constexpr int kBarQFull = 0;                       // [2]  TMA -> MMA: Q tile landed
constexpr int kBarQEmpty = 2;                      // [2]  MMA -> TMA: last QK^T of the item is done
constexpr int kBarKVFull = 4;                      // [kStages]
constexpr int kBarKVEmpty = kBarKVFull + kStages;  // [kStages]
constexpr int kBarSFull = kBarKVEmpty + kStages;   // [2]  MMA -> softmax: S_t ready
constexpr int kBarPFull = kBarSFull + 2;           // [2]  softmax -> MMA: P_t written, O_t rescaled
constexpr int kBarOFull = kBarPFull + 2;           // [2]  MMA -> softmax: last PV of the item is done
constexpr int kBarQRot = kBarOFull + 2;            // [2]  softmax -> MMA: the Q tile has been rotated in place (RoPE)
constexpr int kNumBars = kBarQRot + 2;
constexpr int kSmemMisc = kSmemBars + kNumBars * 8;   // tmem base word, abort flag
constexpr int kSmemTotal = kSmemMisc + 16;
constexpr int kSmemLaunch = kSmemTotal + 1024;        // slack to align the base to 1024 B

struct TcParams {
    void* out;
    float* lse;
    int B, Hq, Hkv, Lq, Lk;
    int64_t os[3];
    int causal;
    float scale;
    float scale_log2;
    float inv_scale_log2;
    float inv_scale;     // additive mask values are divided by the scale before they join S
    const void* mask;    // [B, Hq, Lq, Lk] with element strides ms (0 = broadcast), or null
    int mask_kind;       // 1 bool (true = attend), 2 additive in the tensors' dtype, 3 additive fp32
    int64_t ms[4];
    int* status;
    // rotary embedding of the queries in the prologue (ROPE kernels): cos / sin [rows, 128] in the
    // tensors' dtype, read at row rope_pos0 + query index
    const void* rope_cos;
    const void* rope_sin;
    int64_t rope_pos0;
    int nq;      // 256-row query blocks per (batch, head)
    int npair;   // ceil(nq / 2)
    int units;   // B * Hq * npair * nsplit
    // Split keys (few query blocks against a long key range): a unit covers kv tiles
    // [split * split_tiles, (split + 1) * split_tiles) only, and writes its normalised partial
    // output and its log-sum-exp to scratch rows split * lq_pad + row; a second kernel merges them.
    int nsplit;         // 1 = off
    int split_tiles;    // kv tiles per split
    int split_units;    // units per split = B * Hq * npair
    int lq_pad;         // nq * 256
    int64_t lse_bh;     // lse elements per (batch, head): Lq, or nsplit * lq_pad
    // Packed GQA groups (PACK): an item is one (batch, kv head); its 256 rows are the group's query heads,
    // 2^pack_shift rows each (Lq <= 2^pack_shift), so a few query positions of 2, 4 or 8 heads fill both
    // tiles against one pass over K/V.  Units are (split, batch, kv head); lq_pad = 2^pack_shift.
    int pack_shift;
    // A bool mask that is one row of keys per batch element (sequences padded to a common length), MASK
    // kernels only: kv_len[b] = 1 + the last key of batch element b that may be attended (Lk when it has none:
    // such rows end as NaN through the ordinary mask path), key_prefix[b] != 0 when every key before it may
    // be.  An item visits the kv tiles below kv_len[b] only, and a prefix mask is applied as a sequence
    // length (the tile on the boundary is cut like a ragged last tile) without reading the mask again.
    const int* kv_len;
    const int* key_prefix;
    // A mask shared by every batch element and head ([Lq, Lk]) that turns out to be the causal mask written
    // out (true / 0 where key <= query, false / -inf elsewhere): *mask_is_causal != 0, set by a scan kernel
    // before the launch.  The MASK kernel then runs as the causal kernel does (no kv tile above the diagonal,
    // the diagonal tile cut by position) and does not read the mask.
    const int* mask_is_causal;
    int kv_len_if_causal;   // kv_len holds what the causal check found per batch element: valid only if *mask_is_causal
    // Two launches for one call, of which the device picks one: this launch returns at once unless
    // (*gate != 0) == (gate_want != 0).  (A mask that may be the causal mask: the causal kernel runs if it is,
    // the masked kernel if it is not.)
    const int* gate;
    int gate_want;
};

// One work item = one 256-row query block of one (batch, head).
struct Item {
    int b, h, hk;
    int start[2];  // first query row of each 128-row tile
    int ntile[2];  // kv tiles each query tile visits (0 = tile is past the end of the sequence)
    int n;         // max of the two
    int kv0;       // first kv tile (0 unless the keys are split)
    int orow;      // output row offset (split * lq_pad)
    int lk;        // keys this item may see (MASK kernels with kv_len: the batch element's; else Lk)
};

__device__ __forceinline__ int kv_tiles_for(const TcParams& p, int start, int lk, bool causal) {
    if (start >= p.Lq) return 0;
    int last = lk;
    if (causal) last = min(last, min(p.Lq, start + BM));  // keys 0..row
    return (last + BN - 1) / BN;
}

// Static persistent schedule.  A unit pairs the query blocks (nq-1-pair) and (pair) of one
// head: under a causal mask their kv-tile counts add up to the same total for every pair,
// so handing out units round-robin keeps the CTAs balanced without an atomic work queue,
// and the query blocks of one head (and the heads of one GQA group, which are adjacent
// units) run at the same time, so their K/V tiles are L2 hits.
// `seq` counts items of this CTA: unit = blockIdx.x + (seq/2)*gridDim.x, half = seq & 1.
template <bool SPLIT, bool PACK, bool MASK>
__device__ __forceinline__ bool get_item(const TcParams& p, int seq, Item* it) {
    it->lk = p.Lk;
    if (PACK) {
        int unit = int(blockIdx.x) + seq * int(gridDim.x);
        if (unit >= p.units) return false;
        const int split = SPLIT ? unit / p.split_units : 0;
        unit -= split * p.split_units;
        it->kv0 = split * p.split_tiles;
        it->orow = split * p.lq_pad;
        it->b = unit / p.Hkv;
        it->hk = unit - it->b * p.Hkv;
        it->h = it->hk * (p.Hq / p.Hkv);   // first head of the group
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            it->start[t] = 0;              // every row of the item is a query position below 2^pack_shift
            it->ntile[t] = kv_tiles_for(p, 0, p.Lk, p.causal != 0);
            if (SPLIT) it->ntile[t] = min(max(it->ntile[t] - it->kv0, 0), p.split_tiles);
        }
        it->n = it->ntile[0];
        return true;
    }
    int unit = int(blockIdx.x) + (seq >> 1) * int(gridDim.x);
    if (unit >= p.units) return false;
    // the split is the slowest index: CTAs that run at the same time work on neighbouring heads of
    // the same key range, so the heads of a GQA group still find their K/V tiles in L2
    const int split = SPLIT ? unit / p.split_units : 0;
    unit -= split * p.split_units;
    it->kv0 = split * p.split_tiles;
    it->orow = split * p.lq_pad;
    const int hb = unit / p.npair;
    const int pair = unit - hb * p.npair;
    const int hi = p.nq - 1 - pair;
    const int qblk = (seq & 1) ? pair : hi;
    it->b = hb / p.Hq;
    it->h = hb - it->b * p.Hq;
    it->hk = it->h / (p.Hq / p.Hkv);
    const bool dup = (seq & 1) && pair == hi;  // odd block count: the middle block has no partner
    const bool causal = p.causal != 0 || (MASK && p.mask_is_causal && __ldg(p.mask_is_causal) != 0);
    if (MASK && p.kv_len && (!p.kv_len_if_causal || causal)) it->lk = __ldg(p.kv_len + it->b);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        it->start[t] = qblk * (kTilesPerCta * BM) + t * BM;
        it->ntile[t] = dup ? 0 : kv_tiles_for(p, it->start[t], MASK ? it->lk : p.Lk, causal);
        if (SPLIT) it->ntile[t] = min(max(it->ntile[t] - it->kv0, 0), p.split_tiles);
    }
    it->n = max(it->ntile[0], it->ntile[1]);
    return true;
}

// True when one of the 16 bytes is zero (bool mask bytes: zero = masked out).
__device__ __forceinline__ bool any_zero_byte(const uint4& w) {
    const uint32_t t = ((w.x - 0x01010101u) & ~w.x) | ((w.y - 0x01010101u) & ~w.y) |
                       ((w.z - 0x01010101u) & ~w.z) | ((w.w - 0x01010101u) & ~w.w);
    return (t & 0x80808080u) != 0;
}

// MASK: an explicit attn_mask is applied (a separate instantiation: the unmasked kernel pays
// nothing for it, not even registers).  ROPE: the query tile is rotated in shared memory, by the
// softmax warps that own its rows, between its TMA load and the first QK^T (head dim 128).
// SPLIT: units cover a piece of the key range and write partial results (its own instantiation as
// well: an index added on the softmax chain costs the unsplit kernel 2-3 %).
// LENS: the kernel without mask code, but with a key count per batch element (p.kv_len): what a mask that
// turned out to be lengths, or the causal mask over padded sequences, runs on.
template <bool BF16, bool MASK, int HD, bool ROPE = false, bool SPLIT = false, bool PACK = false, bool LENS = false>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
               const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto bar = [&](int i) { return smem_base + kSmemBars + 8u * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kSmemMisc + 4);

    constexpr int kChunks = HD / 64;                 // 64-element slabs of the head dim
    constexpr uint32_t kLoadBytes = kChunks * kChunkBytes;   // bytes one Q / K / V tile brings in
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (p.gate && (__ldg(p.gate) != 0) != (p.gate_want != 0)) return;   // the other launch of the pair does this call

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool four = (i >= kBarPFull && i < kBarPFull + 2) || i >= kBarQRot;
            const bool two = i >= kBarKVFull && i < kBarKVFull + kStages;
            // one arrival per softmax warp / per entry of a K/V pair / else one commit or TMA
            mbar_init(bar(i), four ? 4u : (two ? 2u : 1u));
        }
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_base + kSmemMisc, kTmemCols);
        tmem_relinquish();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_o);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp >= kMmaWarp) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
      if (warp == kLoadWarp) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            bool ok = true;
            // K/V tiles are loaded in the order the MMAs use them, across items:
            //   K0 | V0 K1 | V1 K2 | ... | V_last K0' | V0' K1' | ...
            // Entry r goes to pair (r+1)/2: an odd entry (V) opens a pair, the following even
            // entry (K of the next step, or K0 of the next item) completes it.  One full and one
            // empty barrier per pair: the issuing thread pays one wait and one commit per step.
            // Each entry arrives once on the pair's full barrier (count 2) with its own byte
            // count; the V-less first pair and the K-less last pair get a plain arrival instead.
            int r = 0;
            uint32_t qcnt[2] = {0, 0};  // items that used query tile t
            auto load_entry = [&](const CUtensorMap* map, int row, int hk, int b) -> bool {
                const int g = (r + 1) >> 1, slot = g & 1;
                const uint32_t full = bar(kBarKVFull + slot);
                if ((r & 1) || r == 0) {  // first entry of the pair: the slot must have been released
                    if (!mbar_wait(bar(kBarKVEmpty + slot), ((g >> 1) & 1) ^ 1u, abort_flag, 2)) return false;
                    if (r == 0) mbar_arrive(full);
                }
                mbar_arrive_expect_tx(full, kLoadBytes);
                const uint32_t dst = smem_base + kSmemKV + slot * kPairBytes + ((r & 1) ? 0 : kTileBytes);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) tma_load_4d(dst + c * kChunkBytes, map, full, 64 * c, row, hk, b);
                ++r;
                return true;
            };
            Item it;
            for (int seq = 0; ok && get_item<SPLIT, PACK, MASK || LENS>(p, seq, &it); ++seq) {
                if (it.n == 0) continue;
                const int kv0 = SPLIT ? it.kv0 : 0;
                ok = load_entry(&map_k, kv0 * BN, it.hk, it.b);  // K0 completes the previous item's last pair
                if (!ok) break;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (ok && it.ntile[t] > 0) {
                        // the previous item's last QK^T on this Q buffer has completed
                        ok = mbar_wait(bar(kBarQEmpty + t), (qcnt[t] & 1u) ^ 1u, abort_flag, 0 + t);
                        if (!ok) break;
                        ++qcnt[t];
                        mbar_arrive_expect_tx(bar(kBarQFull + t), kLoadBytes);
                        const uint32_t dst = smem_base + kSmemQ + t * kTileBytes;
#pragma unroll
                        for (int c = 0; c < kChunks; ++c)
                            tma_load_4d(dst + c * kChunkBytes, &map_q, bar(kBarQFull + t), 64 * c, it.start[t],
                                        PACK ? it.h + (t << (7 - p.pack_shift)) : it.h, it.b);   // (PACK: a box of several heads)
                    }
                }
                for (int x = 1; ok && x < 2 * it.n; ++x)
                    ok = load_entry((x & 1) ? &map_v : &map_k, (kv0 + (x >> 1)) * BN, it.hk, it.b);
            }
            if (ok && r > 0) mbar_arrive(bar(kBarKVFull + ((r >> 1) & 1)));  // the last pair has no K
        }
      } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_f16(BF16 ? 1 : 0, BM, BN, false, false);
            constexpr uint32_t idesc_pv = instr_desc_f16(BF16 ? 1 : 0, BM, HD, false, true);
            auto issue_qk = [&](int t, int pair) {
                const uint32_t qa = smem_base + kSmemQ + t * kTileBytes;
                const uint32_t ka = smem_base + kSmemKV + (pair & 1) * kPairBytes + kTileBytes;
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t off = c * kChunkBytes + i * 32;  // 16 elements = 32 B
                        mma_ss(tmem + kColS + t * 128, smem_desc_sw128(qa + off, 16, 1024),
                               smem_desc_sw128(ka + off, 16, 1024), idesc_qk, (c | i) ? 1u : 0u);
                    }
            };
            auto issue_pv = [&](int t, int pair, bool acc) {
                const uint32_t va = smem_base + kSmemKV + (pair & 1) * kPairBytes;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // 16 keys = 16 rows of 128 B inside each 64-wide half of the head dim
                    mma_ts(tmem + kColO + t * 128, tmem + kColS + t * 128 + ks * 8,
                           smem_desc_sw128(va + ks * 16 * 128, kChunkBytes, 1024), idesc_pv,
                           (acc || ks) ? 1u : 0u);
                }
            };
            bool ok = true;
            int G = 0;                  // pair that holds the current item's K0 (and the previous item's last V)
            bool have = false;          // pair G has already been waited for (by the previous item's last step)
            uint32_t qcnt[2] = {0, 0};   // items that used tile t (Q / O barriers)
            uint32_t pcnt[2] = {0, 0};   // softmax iterations of tile t so far (P barrier)
            Item it;
            for (int seq = 0; ok && get_item<SPLIT, PACK, MASK || LENS>(p, seq, &it); ++seq) {
                if (it.n == 0) continue;
                if (!have) ok = mbar_wait(bar(kBarKVFull + (G & 1)), (G >> 1) & 1, abort_flag, 3);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (ok && it.ntile[t] > 0) {
                        ok = mbar_wait(bar((ROPE ? kBarQRot : kBarQFull) + t), qcnt[t] & 1u, abort_flag, 4 + t);
                        if (ok) {
                            tc_fence_after_sync();
                            issue_qk(t, G);
                            tc_commit(bar(kBarSFull + t));
                            if (it.ntile[t] == 1) tc_commit(bar(kBarQEmpty + t));
                        }
                    }
                }
                if (!ok) break;
                tc_commit(bar(kBarKVEmpty + (G & 1)));  // after the previous item's last PV and these QK^T
                for (int j = 0; ok && j < it.n; ++j) {
                    const int g = G + j + 1;  // (V_j, K_j+1)
                    ok = mbar_wait(bar(kBarKVFull + (g & 1)), (g >> 1) & 1, abort_flag, 3);
                    if (!ok) break;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (ok && j < it.ntile[t]) {
                            ok = mbar_wait(bar(kBarPFull + t), pcnt[t] & 1u, abort_flag, 6 + t);
                            if (!ok) break;
                            ++pcnt[t];
                            // (the first PV of an item overwrites O_t: these warps read the previous
                            // item's O_t out before they started on this item's first S tile, so the
                            // P barrier covers that too)
                            tc_fence_after_sync();
                            issue_pv(t, g, j > 0);
                            if (j + 1 < it.ntile[t]) {
                                issue_qk(t, g);
                                tc_commit(bar(kBarSFull + t));
                                if (j + 2 == it.ntile[t]) tc_commit(bar(kBarQEmpty + t));
                            } else {
                                tc_commit(bar(kBarOFull + t));
                            }
                        }
                    }
                    if (!ok) break;
                    // the last pair of the item also holds the next item's K0: released there
                    if (j + 1 < it.n) tc_commit(bar(kBarKVEmpty + (g & 1)));
                }
#pragma unroll
                for (int t = 0; t < 2; ++t)
                    if (it.ntile[t] > 0) ++qcnt[t];
                G += it.n;
                have = true;
            }
        }
        __syncwarp();
      }
    } else {
        // ------------------------------ softmax + epilogue --------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int t = warp >> 2;
        const int wq = warp & 3;
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + kColS + t * 128;
        const uint32_t o_addr = tmem + lane_base + kColO + t * 128;
        const uint32_t o_stage = smem_base + kSmemO + warp * kOStageBytes;
        const float c2 = p.scale_log2;
        bool ok = true;
        uint32_t scnt = 0;  // S tiles consumed so far
        uint32_t ocnt = 0;  // items finished so far
        Item it;
        for (int seq = 0; ok && get_item<SPLIT, PACK, MASK || LENS>(p, seq, &it); ++seq) {
            const int nt = it.ntile[t];
            if (nt == 0) continue;
            const int lk_item = (MASK || LENS) ? it.lk : p.Lk;
            const bool dyn_causal = MASK && p.mask_is_causal && __ldg(p.mask_is_causal) != 0;
            const bool causal = p.causal != 0 || dyn_causal;
            const bool mask_off = dyn_causal || (MASK && p.key_prefix && __ldg(p.key_prefix + it.b) != 0);   // position or length says it all
            // PACK: row r of the tile is query position r mod 2^pack_shift of head r >> pack_shift of the group
            const int row_q = PACK ? ((wq * 32 + lane) & ((1 << p.pack_shift) - 1)) : it.start[t] + wq * 32 + lane;
            const int head_q = PACK ? it.h + ((t * BM + wq * 32) >> p.pack_shift) : it.h;   // (a warp's 32 rows: one head)
            if (ROPE) {
                // this lane's row of the freshly landed Q tile, rotated in place: 16-byte unit u of row r
                // sits at u ^ (r & 7) in each 64-column slab; columns d and d + 64 share the offset
                // The warp rotates its 32 rows four at a time, eight lanes per row: lane l takes
                // 16-byte unit (l & 7) of row 4g + (l >> 3) in both 64-column slabs.  The table rows
                // are then read 128 contiguous bytes per row (a lane per row would touch 32 rows
                // per instruction).  All 32 table loads are issued before the wait for the tile, so
                // that their latency runs under the tile's own.
                const int u = lane & 7;
                const uint32_t tile = smem_base + kSmemQ + t * kTileBytes;
                uint4 c1[8], s1[8], c2[8], s2[8];
                {
                    const int64_t pos_w = p.rope_pos0 + it.start[t] + wq * 32;
                    const uint4* cs = static_cast<const uint4*>(p.rope_cos);
                    const uint4* sn = static_cast<const uint4*>(p.rope_sin);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = 4 * i + (lane >> 3);                         // row within the warp's 32
                        const bool live = it.start[t] + wq * 32 + rr < p.Lq;
                        const int64_t trow = live ? (pos_w + rr) * (HD / 8) : 0;   // rows past the end: any valid row
                        c1[i] = __ldg(cs + trow + u);
                        s1[i] = __ldg(sn + trow + u);
                        c2[i] = __ldg(cs + trow + 8 + u);
                        s2[i] = __ldg(sn + trow + 8 + u);
                    }
                }
                ok = mbar_wait(bar(kBarQFull + t), ocnt & 1u, abort_flag, 18 + t);
                if (!ok) break;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = wq * 32 + 4 * i + (lane >> 3);        // row within the tile
                    const uint32_t addr = tile + r * 128 + uint32_t((u ^ (r & 7)) << 4);
                    uint4 x1, x2;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x1.x), "=r"(x1.y), "=r"(x1.z), "=r"(x1.w) : "r"(addr));
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x2.x), "=r"(x2.y), "=r"(x2.z), "=r"(x2.w) : "r"(addr + kChunkBytes));
                    rope_rotate8<BF16>(x1, x2, c1[i], s1[i], c2[i], s2[i]);
                    st_shared_v4(addr, x1);
                    st_shared_v4(addr + kChunkBytes, x2);
                }
                fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarQRot + t));
            }
            // Explicit attn_mask (csrc/ops/attention_ops.cpp:117-126): this thread's row of it, 128
            // entries per kv tile.  Bool: false -> -inf.  Additive: S is still unscaled here, so the
            // mask value joins it divided by the scale.  Rows past the end reuse the last row.
            const char* mrow = nullptr;
            // Staged reading of a mask whose rows are contiguous along the keys.  A lane owns a query
            // row, so reading its own row touches 32 rows (cache lines) per instruction and the
            // lines do not survive in L1 until the lane comes back for their other 16-byte pieces.
            // Instead the warp reads its 32 rows 128 contiguous bytes at a time (8 lanes per row,
            // 4 rows per instruction), passes them through its 4 KB staging buffer (the one the O
            // store uses at the end of the item) and each lane picks its own row up from there.
            // A "slice" is 128 bytes of every row: 128 / 64 / 32 keys for 1 / 2 / 4-byte masks.
            const char* mask_bh = nullptr;
            int64_t mpitch = 0;
            int mesz = 1;
            bool mfast = false, mbcast = false;
            if (MASK) {
                mesz = p.mask_kind == 1 ? 1 : (p.mask_kind == 2 ? 2 : 4);
                mask_bh = static_cast<const char*>(p.mask) + (int64_t(it.b) * p.ms[0] + int64_t(it.h) * p.ms[1]) * mesz;
                mpitch = p.ms[2] * mesz;
                mrow = mask_bh + int64_t(min(row_q, p.Lq - 1)) * mpitch;
                // (a row shared by every query, pitch 0, is one line per instruction as it is)
                mfast = p.ms[3] == 1 && mpitch != 0 && (mpitch & 15) == 0 && (reinterpret_cast<uintptr_t>(mask_bh) & 15u) == 0;
                if (mfast) {
                    if (lane == 0) tma_store_wait_read();   // the previous item's O store has read the buffer
                    __syncwarp();
                }
                // one bool row for every query (a key-padding mask): its 128 bytes per kv tile are
                // fetched before the wait for S, so that their latency is not part of the tile's chain
                mbcast = p.mask_kind == 1 && p.ms[3] == 1 && mpitch == 0 && (reinterpret_cast<uintptr_t>(mask_bh) & 15u) == 0;
            }
            const int mu = lane & 7, mrs = lane >> 3;
            auto mask_ldg = [&](int col0, int r, uint4 (&w)[8]) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int grow = min(it.start[t] + wq * 32 + 4 * i + mrs, p.Lq - 1);
                    w[i] = __ldg(reinterpret_cast<const uint4*>(mask_bh + int64_t(grow) * mpitch + int64_t(col0) * mesz + r * 128) + mu);
                }
            };
            auto mask_sts = [&](const uint4 (&w)[8]) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = 4 * i + mrs;
                    st_shared_v4(o_stage + row * 128 + uint32_t((mu ^ (row & 7)) << 4), w[i]);
                }
            };
            auto mask_lds = [&](int v) {
                uint4 x;
                const uint32_t addr = o_stage + lane * 128 + uint32_t((v ^ (lane & 7)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "r"(addr));
                return x;
            };
            // slice r of the staged mask (already in the staging buffer) joins this lane's scores
            auto mask_apply_slice = [&](uint32_t (&s)[BN], int r) {
                if (p.mask_kind == 1) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const uint4 w = mask_lds(v);
                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (((ww[e >> 2] >> (8 * (e & 3))) & 0xffu) == 0) s[16 * v + e] = 0xff800000u;
                    }
                } else if (p.mask_kind == 2) {
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        if (rr != r) continue;
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const uint4 w = mask_lds(v);
                            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {   // two keys per packed FMA
                                const int i0 = 64 * rr + 8 * v + 2 * e;
                                const float2 r2 = ffma2(pair16_to_f32<BF16>(ww[e]), make_float2(p.inv_scale, p.inv_scale),
                                                        make_float2(__uint_as_float(s[i0]), __uint_as_float(s[i0 + 1])));
                                s[i0] = __float_as_uint(r2.x);
                                s[i0 + 1] = __float_as_uint(r2.y);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) {
                        if (rr != r) continue;
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const uint4 w = mask_lds(v);
                            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int i0 = 32 * rr + 4 * v + 2 * e;
                                const float2 r2 = ffma2(make_float2(__uint_as_float(ww[2 * e]), __uint_as_float(ww[2 * e + 1])),
                                                        make_float2(p.inv_scale, p.inv_scale),
                                                        make_float2(__uint_as_float(s[i0]), __uint_as_float(s[i0 + 1])));
                                s[i0] = __float_as_uint(r2.x);
                                s[i0 + 1] = __float_as_uint(r2.y);
                            }
                        }
                    }
                }
            };
            // the slices after the first: `w` holds slice 1, fetched before the wait for S
            auto mask_apply_staged = [&](uint32_t (&s)[BN], int col0, uint4 (&w)[8]) {
                mask_apply_slice(s, 0);
                for (int r = 1; r < mesz; ++r) {
                    __syncwarp();                       // every lane has read slice r-1
                    mask_sts(w);
                    if (r + 1 < mesz) mask_ldg(col0, r + 1, w);
                    __syncwarp();
                    mask_apply_slice(s, r);
                }
                __syncwarp();
            };
            auto apply_mask = [&](uint32_t (&s)[BN], int col0) {
                const int ncols = min(BN, p.Lk - col0);
                const bool vec = p.ms[3] == 1 && ncols == BN;
                if (p.mask_kind == 1) {
                    const unsigned char* mp = reinterpret_cast<const unsigned char*>(mrow) + int64_t(col0) * p.ms[3];
                    if (vec && (reinterpret_cast<uintptr_t>(mp) & 15u) == 0) {
#pragma unroll
                        for (int v = 0; v < BN / 16; ++v) {
                            const uint4 w = __ldg(reinterpret_cast<const uint4*>(mp) + v);
                            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                if (((ww[e >> 2] >> (8 * (e & 3))) & 0xffu) == 0) s[16 * v + e] = 0xff800000u;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < BN; ++i)
                            if (i < ncols && mp[int64_t(i) * p.ms[3]] == 0) s[i] = 0xff800000u;
                    }
                } else if (p.mask_kind == 2) {
                    const uint16_t* mp = reinterpret_cast<const uint16_t*>(mrow) + int64_t(col0) * p.ms[3];
                    if (vec && (reinterpret_cast<uintptr_t>(mp) & 15u) == 0) {
#pragma unroll
                        for (int v = 0; v < BN / 8; ++v) {
                            const uint4 w = __ldg(reinterpret_cast<const uint4*>(mp) + v);
                            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {   // two keys per packed FMA
                                const int i0 = 8 * v + 2 * e;
                                const float2 r2 = ffma2(pair16_to_f32<BF16>(ww[e]), make_float2(p.inv_scale, p.inv_scale),
                                                        make_float2(__uint_as_float(s[i0]), __uint_as_float(s[i0 + 1])));
                                s[i0] = __float_as_uint(r2.x);
                                s[i0 + 1] = __float_as_uint(r2.y);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < BN; ++i)
                            if (i < ncols)
                                s[i] = __float_as_uint(fmaf(from16<BF16>(mp[int64_t(i) * p.ms[3]]), p.inv_scale,
                                                            __uint_as_float(s[i])));
                    }
                } else {
                    const float* mp = reinterpret_cast<const float*>(mrow) + int64_t(col0) * p.ms[3];
                    if (vec && (reinterpret_cast<uintptr_t>(mp) & 15u) == 0) {
#pragma unroll
                        for (int v = 0; v < BN / 4; ++v) {
                            const float4 w = __ldg(reinterpret_cast<const float4*>(mp) + v);
                            s[4 * v + 0] = __float_as_uint(fmaf(w.x, p.inv_scale, __uint_as_float(s[4 * v + 0])));
                            s[4 * v + 1] = __float_as_uint(fmaf(w.y, p.inv_scale, __uint_as_float(s[4 * v + 1])));
                            s[4 * v + 2] = __float_as_uint(fmaf(w.z, p.inv_scale, __uint_as_float(s[4 * v + 2])));
                            s[4 * v + 3] = __float_as_uint(fmaf(w.w, p.inv_scale, __uint_as_float(s[4 * v + 3])));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < BN; ++i)
                            if (i < ncols)
                                s[i] = __float_as_uint(fmaf(mp[int64_t(i) * p.ms[3]], p.inv_scale, __uint_as_float(s[i])));
                    }
                }
            };
            float m = -INFINITY, m_next = -INFINITY, l = 0.f;
            bool move_ref = false;
            for (int j = 0; j < nt; ++j) {
                uint4 mw[8];
                bool staged = false, early = false;
                if (MASK) {
                    // these warps are idle until S arrives: slice 0 of this step's mask goes to the staging
                    // buffer now, slice 1 stays in flight across the wait
                    staged = mfast && !mask_off && (j + 1) * BN <= p.Lk;
                    if (staged) {
                        uint4 w0[8];
                        mask_ldg(j * BN, 0, w0);
                        if (mesz > 1) mask_ldg(j * BN, 1, mw);
                        mask_sts(w0);
                        __syncwarp();
                    }
                    early = mbcast && !mask_off && (j + 1) * BN <= p.Lk;
                    if (early) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) mw[v] = __ldg(reinterpret_cast<const uint4*>(mask_bh + j * BN) + v);
                    }
                }
                ok = mbar_wait(bar(kBarSFull + t), scnt & 1u, abort_flag, 10 + t);
                if (!ok) break;
                ++scnt;
                tc_fence_after_sync();
                // O_t *= alpha (per row), in TMEM.  PV_t(j-1) has completed (S_t(j) was committed
                // after it) and PV_t(j) waits for this tile's P barrier, so O_t is quiescent here.
                auto rescale_o = [&](float alpha) {
#pragma unroll 1
                    for (int c = 0; c < HD / 16; ++c) {
                        uint32_t o[16];
                        tmem_ld16(o_addr + 16 * c, o);
                        tmem_wait_ld();
                        tmem_ld_fence16(o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st16(o_addr + 16 * c, o);
                    }
                };
                // Only the item's first tile looks for its row max before exponentiating: that pass
                // heads the tile's dependency chain (S ready -> P ready -> next S ...).  Later tiles
                // exponentiate against the reference m they are given, and the row sum they get
                // tells whether m was good enough:
                //   sum > kRedoSum (or not finite): a P could overflow.  P has not been stored yet,
                //       so S_t is intact: load it again, take the row's max as m, and redo (rare)
                //   sum > kRescaleSum: m moves up by log2(sum)/c from the next tile on
                // Any reference gives the exact O/l as long as l and O are rescaled when it moves,
                // so m need not be the true max.
                if (j > 0 && move_ref) {  // voted on after the previous hand-over, while waiting for this S
                    const float alpha = ex2_approx((m - m_next) * c2);  // 1 for rows that keep theirs
                    l *= alpha;
                    rescale_o(alpha);
                    m = m_next;
                }
                uint32_t pk[BN / 2];
                float l_tile;
                bool bad = false;
#pragma unroll 1
                for (int attempt = 0;; ++attempt) {
                    uint32_t s[BN];
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        tmem_ld32(s_addr + 32 * c, reinterpret_cast<uint32_t(&)[32]>(s[32 * c]));
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld_fence32(reinterpret_cast<uint32_t(&)[32]>(s[32 * c]));
                    const int col0 = SPLIT ? (it.kv0 + j) * BN : j * BN;
                    const bool need_mask = (causal && col0 + BN - 1 > it.start[t]) || (col0 + BN > lk_item);
                    if (need_mask) {
                        const int limit = (causal ? min(row_q, lk_item - 1) : lk_item - 1) - col0;
#pragma unroll
                        for (int i = 0; i < BN; ++i)
                            if (i > limit) s[i] = 0xff800000u;  // -inf
                    }
                    if (MASK && !mask_off) {
                        if (staged && attempt == 0) {
                            mask_apply_staged(s, col0, mw);
                        } else if (early) {
#pragma unroll
                            for (int v = 0; v < 8; ++v) {
                                if (!any_zero_byte(mw[v])) continue;   // these 16 keys are all visible
                                const uint32_t ww[4] = {mw[v].x, mw[v].y, mw[v].z, mw[v].w};
#pragma unroll
                                for (int e = 0; e < 16; ++e)
                                    if (((ww[e >> 2] >> (8 * (e & 3))) & 0xffu) == 0) s[16 * v + e] = 0xff800000u;
                            }
                        } else {
                            apply_mask(s, col0);
                        }
                    }
                    if (j == 0 || attempt == 1) {
                        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                        for (int i = 0; i < BN; i += 4) {
                            mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                            mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                        }
                        float m_new = (j == 0 || bad) ? fmaxf(mx0, mx1) : m;
                        // every key so far masked out for this row: any finite reference will do (all
                        // its P are 0); a row that stays that way ends as 0/0 = NaN like the reference
                        if (MASK && m_new == -INFINITY) m_new = 0.f;
                        if (j > 0) {
                            const float alpha = ex2_approx((m - m_new) * c2);
                            l *= alpha;
                            rescale_o(alpha);
                        }
                        m = m_new;
                    }
                    // two columns per instruction on the FMA pipe (fp32x2 FMA / ADD)
                    const float neg_m = -m * c2;
                    const float2 c22 = make_float2(c2, c2), nm2 = make_float2(neg_m, neg_m);
                    float2 ls0 = make_float2(0.f, 0.f), ls1 = make_float2(0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < BN / 2; ++i) {
                        const float2 x = ffma2(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), c22, nm2);
                        const float p0 = ex2_approx(x.x), p1 = ex2_approx(x.y);
                        if (i & 1) ls1 = fadd2(ls1, make_float2(p0, p1));
                        else ls0 = fadd2(ls0, make_float2(p0, p1));
                        pk[i] = pack16<BF16>(p0, p1);
                    }
                    l_tile = (ls0.x + ls0.y) + (ls1.x + ls1.y);
                    if (j == 0 || attempt == 1) break;
                    bad = !(l_tile <= kRedoSum);
                    if (!__any_sync(0xffffffffu, bad)) break;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c)  // P_t over the first 64 columns of S_t
                    tmem_st16(s_addr + 16 * c, reinterpret_cast<uint32_t(&)[16]>(pk[16 * c]));
                l += l_tile;
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarPFull + t));
                // off the chain: these warps now wait for the tensor core anyway
                m_next = l_tile > kRescaleSum ? m + lg2_approx(l_tile) * p.inv_scale_log2 : m;
                move_ref = __any_sync(0xffffffffu, m_next != m);
            }
            if (!ok) break;
            ok = mbar_wait(bar(kBarOFull + t), ocnt & 1u, abort_flag, 16 + t);
            if (!ok) break;
            ++ocnt;
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            const bool live = row_q < p.Lq;
            // O leaves through shared memory and a TMA store: a lane owns a row, so direct global
            // stores would touch 32 cache lines per instruction.  Two halves of 64 columns share
            // the warp's 4 KB staging buffer (128-byte swizzle: 16-byte chunk c of row r sits at
            // chunk c ^ (r & 7)); rows past the end of the sequence are clipped by the tensor map.
            const int row_w = PACK ? ((wq * 32) & ((1 << p.pack_shift) - 1)) : it.start[t] + wq * 32;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(o_addr + 32 * c, o);
                tmem_wait_ld();
                tmem_ld_fence32(o);
                if ((c & 1) == 0) {
                    if (lane == 0) tma_store_wait_read();  // the previous store has read the buffer
                    __syncwarp();
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 w;
                    w.x = pack16<BF16>(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                    w.y = pack16<BF16>(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                    w.z = pack16<BF16>(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                    w.w = pack16<BF16>(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                    st_shared_v4(o_stage + lane * 128 + (((4 * (c & 1) + v) ^ (lane & 7)) << 4), w);
                }
                if (c & 1) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row_w < p.Lq) {
                        tma_store_4d(&map_o, o_stage, 64 * (c >> 1), (SPLIT ? it.orow : 0) + row_w, head_q, it.b);
                        tma_store_commit();
                    }
                }
            }
            if (p.lse && live)
                p.lse[SPLIT ? (int64_t(it.b) * p.Hq + head_q) * p.lse_bh + it.orow + row_q
                            : (int64_t(it.b) * p.Hq + head_q) * p.Lq + row_q] = m * p.scale + logf(l);
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
        // 0x40000000 | one bit per wait that was still pending.  The grid is persistent (one wave),
        // so a broken launch costs every CTA one time limit in parallel, not one after another.
        *p.status = *abort_flag;
        __threadfence_system();
    }
}

// ---- key-padding masks: the length each batch element's row stands for ---------------------------
// One CTA per batch element over its Lk mask entries (bool: nonzero = valid; additive: 0 = valid, at most
// `masked_below` = removed): kv_len[b] = 1 + the last valid key's index, key_prefix[b] = 1 when every key
// before it is valid too.  A row without a valid key, or an additive row with any other value (a bias, not a
// padding mask), gets kv_len = Lk and key_prefix = 0: the mask is then applied as given.
__global__ void __launch_bounds__(256) key_mask_scan_kernel(const void* __restrict__ mask, int64_t bstride, int Lk, int kind, int bf16,
                                                            float masked_below, int* __restrict__ kv_len,
                                                            int* __restrict__ key_prefix, int* __restrict__ all_prefix) {
    __shared__ int s_last, s_count, s_other;
    if (threadIdx.x == 0) { s_last = -1; s_count = 0; s_other = 0; }
    __syncthreads();
    int last = -1, count = 0;
    bool other = false;
    if (kind == 1) {
        const unsigned char* row = static_cast<const unsigned char*>(mask) + int64_t(blockIdx.x) * bstride;
        if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0 && Lk % 16 == 0) {
            for (int c = int(threadIdx.x); c < Lk / 16; c += 256) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(row) + c);
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if ((ww[j] >> (8 * e)) & 0xffu) { last = 16 * c + 4 * j + e; ++count; }
                }
            }
        } else {
            for (int k = int(threadIdx.x); k < Lk; k += 256)
                if (row[k]) { last = k; ++count; }
        }
    } else {
        for (int k = int(threadIdx.x); k < Lk; k += 256) {
            const int64_t off = int64_t(blockIdx.x) * bstride + k;
            const float f = kind == 3 ? __ldg(static_cast<const float*>(mask) + off)
                                      : (bf16 ? from16<true>(__ldg(static_cast<const uint16_t*>(mask) + off))
                                              : from16<false>(__ldg(static_cast<const uint16_t*>(mask) + off)));
            if (f == 0.f) { last = k; ++count; }
            else if (!(f <= masked_below)) other = true;
        }
    }
    if (last >= 0) atomicMax(&s_last, last);
    if (count) atomicAdd(&s_count, count);
    if (other) atomicOr(&s_other, 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool usable = s_last >= 0 && s_other == 0;
        kv_len[blockIdx.x] = usable ? s_last + 1 : Lk;
        key_prefix[blockIdx.x] = usable && s_count == s_last + 1;
        if (!(usable && s_count == s_last + 1)) atomicAnd(all_prefix, 0);   // (nonzero on entry)
    }
}

// Is a mask the causal mask written out?  Entry (i, j) of batch element b must be visible exactly when
// j <= i and j < len_b.  kind 1: bool, nonzero = visible; kinds 2, 3: additive, 0 = visible, at most
// `masked_below` = removed (-inf, or the most negative finite value of the dtype that some callers write
// instead: with key 0 visible in every row and the scale the launcher checked, exp of such an entry is exactly 0,
// as for -inf); anything else is a bias and fails the check.
//   kv_len == nullptr: one [Lq, Lk] mask for all batch elements, len = Lk (gridDim.y = 1).
//   else: a [B, 1, Lq, Lk] mask over sequences padded on the right; every CTA of batch element b (blockIdx.y)
//   takes len_b from the mask's last row, whose visible entries must be a prefix, and kv_len[b] = len_b.
// *flag is nonzero on entry; any mismatch clears it.  A thread checks 16 consecutive entries of a row at a time
// (16-byte loads when the rows allow).
__global__ void __launch_bounds__(256) causal_check_kernel(const void* __restrict__ mask, int64_t batch_stride, int64_t row_stride,
                                                          int Lq, int Lk, int kind, int bf16, float masked_below,
                                                          int* __restrict__ kv_len, int* __restrict__ flag) {
    __shared__ int s_last, s_count;
    const int b = blockIdx.y;
    const int esz = kind == 1 ? 1 : kind == 2 ? 2 : 4;
    const unsigned char* base = static_cast<const unsigned char*>(mask) + int64_t(b) * batch_stride * esz;
    bool ok = true;
    // visible / removed / neither for the entry at element offset `off` of this batch element
    auto visible = [&](int64_t off) -> bool {
        if (kind == 1) return base[off] != 0;
        const float f = kind == 3 ? reinterpret_cast<const float*>(base)[off]
                                  : (bf16 ? from16<true>(reinterpret_cast<const uint16_t*>(base)[off])
                                          : from16<false>(reinterpret_cast<const uint16_t*>(base)[off]));
        if (f == 0.f) return true;
        if (!(f <= masked_below)) ok = false;
        return false;
    };
    int len = Lk;
    if (kv_len) {
        if (threadIdx.x == 0) { s_last = -1; s_count = 0; }
        __syncthreads();
        int last = -1, count = 0;
        for (int j = int(threadIdx.x); j < Lk; j += 256)
            if (visible(int64_t(Lq - 1) * row_stride + j)) { last = j; ++count; }
        if (last >= 0) atomicMax(&s_last, last);
        if (count) atomicAdd(&s_count, count);
        __syncthreads();
        len = s_last + 1;
        if (len < 1 || s_count != len) ok = false;
        if (blockIdx.x == 0 && threadIdx.x == 0) kv_len[b] = len < 1 ? Lk : len;
    }
    const bool vec = (reinterpret_cast<uintptr_t>(base) & 15u) == 0 && (row_stride * esz) % 16 == 0 && Lk % 16 == 0;
    const int spans = (Lk + 15) / 16;
    const int64_t total = int64_t(Lq) * spans;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total && ok; i += int64_t(gridDim.x) * 256) {
        const int r = int(i / spans), c0 = int(i - int64_t(r) * spans) * 16;
        const int n = max(0, min(16, min(r + 1, len) - c0));   // the first n entries of the span are visible
        const int64_t off = int64_t(r) * row_stride + c0;
        if (vec && kind == 1) {
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(base + off));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 16; ++e) ok = ok && ((((ww[e >> 2] >> (8 * (e & 3))) & 0xffu) != 0) == (e < n));
        } else if (vec && kind == 2) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(base + (off + 8 * h) * 2));
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint16_t bits = uint16_t(ww[e >> 1] >> (16 * (e & 1)));
                    const float f = bf16 ? from16<true>(bits) : from16<false>(bits);
                    ok = ok && (8 * h + e < n ? f == 0.f : f <= masked_below);
                }
            }
        } else {
            for (int e = 0; e < 16 && c0 + e < Lk; ++e) {
                const bool v = visible(off + e);
                ok = ok && v == (e < n);
            }
        }
    }
    if (!__syncthreads_and(ok) && threadIdx.x == 0) atomicAnd(flag, 0);
}

// ---- merge of the split-key partial results ------------------------------------------------
struct CombineParams {
    const uint16_t* part_o;   // [B, Hq, nsplit * lq_pad, HD], each split's output normalised by its own sum
    const float* part_lse;    // [B, Hq, nsplit * lq_pad], natural-log sum of exponentials per split
    void* out;
    float* lse;               // [B, Hq, Lq] or null
    int B, Hq, Lq, Lk, causal, nsplit, split_tiles, lq_pad;
    int64_t os[3];
};

// out[row] = sum_s w_s * part_o[s][row] / sum_s w_s,  w_s = exp(lse_s - max_s lse_s).  A thread owns 8
// columns of a row.  Which splits hold a row follows from the schedule above (a 128-row query tile
// visits the kv tiles below its causal limit), so scratch needs no initialisation.
template <bool BF16, int HD>
__global__ void __launch_bounds__(256) sdpa_tc_combine_kernel(const CombineParams c) {
    constexpr int kPerRow = HD / 8;
    const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
    const int64_t row = idx / kPerRow;
    const int ch = int(idx - row * kPerRow);
    if (row >= int64_t(c.B) * c.Hq * c.Lq) return;
    const int64_t bh = row / c.Lq;
    const int r = int(row - bh * c.Lq);
    const int tile0 = r & ~(BM - 1);
    const int lim = c.causal ? min(c.Lk, min(c.Lq, tile0 + BM)) : c.Lk;
    const int span = c.split_tiles * BN;
    const int live = min(c.nsplit, (lim + span - 1) / span);
    const float* pl = c.part_lse + bh * (int64_t(c.nsplit) * c.lq_pad) + r;
    float mx = -INFINITY;
    for (int sp = 0; sp < live; ++sp) mx = fmaxf(mx, __ldg(pl + int64_t(sp) * c.lq_pad));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float den = 0.f;
    for (int sp = 0; sp < live; ++sp) {
        const float w = expf(__ldg(pl + int64_t(sp) * c.lq_pad) - mx);
        den += w;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(
            c.part_o + ((bh * c.nsplit + sp) * int64_t(c.lq_pad) + r) * HD + 8 * ch));
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(w, from16<BF16>(uint16_t(u[i] & 0xffffu)), acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, from16<BF16>(uint16_t(u[i] >> 16)), acc[2 * i + 1]);
        }
    }
    const float inv = 1.0f / den;
    uint4 o;
    o.x = pack16<BF16>(acc[0] * inv, acc[1] * inv);
    o.y = pack16<BF16>(acc[2] * inv, acc[3] * inv);
    o.z = pack16<BF16>(acc[4] * inv, acc[5] * inv);
    o.w = pack16<BF16>(acc[6] * inv, acc[7] * inv);
    const int b = int(bh / c.Hq), h = int(bh - int64_t(b) * c.Hq);
    uint16_t* dst = static_cast<uint16_t*>(c.out) + b * c.os[0] + h * c.os[1] + r * c.os[2] + 8 * ch;
    *reinterpret_cast<uint4*>(dst) = o;
    if (c.lse && ch == 0) c.lse[row] = mx + logf(den);
}

// ---- host side -------------------------------------------------------------------------
// [B, H, L, D] tensor with element strides st = {B, H, L}
int make_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int L, int D,
             const int64_t* st, int box_rows = BN, int box_heads = 1) {
    return make_tensor_map_bhld(map, base, dtype, B, H, L, D, st, box_rows, box_heads);
}

bool strides_ok(const void* base, const int64_t* st, int B, int H, int L, int D) {
    if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
    if (L > 1 && (st[2] < D || (st[2] * 2) % 16)) return false;
    if (H > 1 && (st[1] <= 0 || (st[1] * 2) % 16)) return false;
    if (B > 1 && (st[0] <= 0 || (st[0] * 2) % 16)) return false;
    return true;
}

// Few query blocks against many keys (a prompt chunk or a handful of new tokens over a long cache):
// B * Hq * npair units cannot fill the GPU, so the key range is cut into `nsplit` pieces of
// `split_tiles` kv tiles.  No mask tensor and no rotary prologue on this route.
//
// Packed groups: with 2, 4 or 8 query heads per kv head and at most 256 / group query positions, the
// group's heads share one item (2^pack_shift rows each), so both tiles are full of live rows and K/V is
// read once per group instead of once per head.
struct SplitPlan { int nsplit, split_tiles, lq_pad, pack_shift; size_t o_bytes, bytes; };

SplitPlan split_plan(const Gpu* g, const paras_sdpa_args& a, bool rope) {
    SplitPlan sp{1, 1 << 28, 0, 0, 0, 0};
    if (a.mask || rope || (a.D != 128 && a.D != 64)) return sp;
    const int group = a.Hkv > 0 && a.Hq % a.Hkv == 0 ? a.Hq / a.Hkv : 1;
    if ((group == 2 || group == 4 || group == 8) && a.Lq * group <= kTilesPerCta * BM)
        sp.pack_shift = group == 2 ? 7 : group == 4 ? 6 : 5;
    const int nq = (a.Lq + kTilesPerCta * BM - 1) / (kTilesPerCta * BM);
    const int64_t units = sp.pack_shift ? int64_t(a.B) * a.Hkv : int64_t(a.B) * a.Hq * ((nq + 1) / 2);
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    if (units * 2 > sms) return sp;
    const int keys = a.causal ? std::min(a.Lk, a.Lq) : a.Lk;
    const int kv = (keys + BN - 1) / BN;
    const int want = int(std::min<int64_t>(std::min<int64_t>(sms / units, kv / 4), 32));
    if (want < 2) return sp;
    const int per = (kv + want - 1) / want;
    const int n = (kv + per - 1) / per;
    if (n < 2) return sp;
    sp.nsplit = n;
    sp.split_tiles = per;
    sp.lq_pad = sp.pack_shift ? 1 << sp.pack_shift : nq * kTilesPerCta * BM;
    const size_t rows = size_t(a.B) * a.Hq * n * sp.lq_pad;
    sp.o_bytes = (rows * a.D * 2 + 255) & ~size_t(255);
    sp.bytes = sp.o_bytes + rows * sizeof(float);
    return sp;
}

}  // namespace

size_t sdpa_tc_workspace_bytes(const Gpu* g, const paras_sdpa_args& a) { return split_plan(g, a, false).bytes; }

// The check of causal_check_kernel for one [Lq, Lk] mask, answered on the host (a copy back and a wait):
// for callers that choose a route by it, as the operator layer does before it picks a backward.
int sdpa_mask_is_causal(Gpu* g, int gpu, const void* mask, int mask_kind, int dtype, int64_t row_stride, int Lq, int Lk,
                        float scale, cudaStream_t s, int* result) {
    *result = 0;
    if (!mask || mask_kind < 1 || mask_kind > 3 || Lq < 1 || Lk < 1) return PARAS_OK;
    void* dev = nullptr;
    int st = paras_b200_malloc_async(gpu, sizeof(int), s, &dev);
    if (st != PARAS_OK) return st;
    int* flag = static_cast<int*>(dev);
    const float masked_below = scale * 1.4426950408889634f * 60000.0f > 1000.0f ? -60000.0f : -INFINITY;
    const int64_t spans = int64_t(Lq) * ((Lk + 15) / 16);
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const unsigned blocks = unsigned(std::min<int64_t>((spans + 255) / 256, int64_t(sms) * 8));
    int host = 0;
    cudaError_t e = cudaMemsetAsync(flag, 1, sizeof(int), s);
    if (e == cudaSuccess) {
        causal_check_kernel<<<blocks, 256, 0, s>>>(mask, 0, row_stride, Lq, Lk, mask_kind, dtype == PARAS_BF16 ? 1 : 0, masked_below,
                                                   nullptr, flag);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(&host, flag, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    const int st2 = paras_b200_free_async(gpu, dev, s);
    if (e != cudaSuccess) return fail(PARAS_E_CUDA, "paras sdpa: mask check failed: %s", cudaGetErrorString(e));
    *result = host != 0;
    return st2;
}

bool sdpa_tc_supported(const Gpu* g, const paras_sdpa_args& a, const char** why) {
    *why = "";
    if (g->cc_major != 10) { *why = "GPU is not compute capability 10.x"; return false; }
    if (a.dtype != PARAS_BF16 && a.dtype != PARAS_F16) { *why = "dtype is not 16-bit"; return false; }
    if (a.D != 128 && a.D != 64) { *why = "head dim is neither 128 nor 64"; return false; }
    if (a.mask && (a.mask_kind < 1 || a.mask_kind > 3)) { *why = "unknown mask kind"; return false; }
    if (a.Lq < 1 || a.Lk < 1) { *why = "empty sequence"; return false; }
    if (!(a.scale > 0.0) || !std::isfinite(a.scale)) { *why = "scale is not positive"; return false; }
    if (a.Hq > 65535 || a.B > 65535) { *why = "batch or heads exceed the grid limit"; return false; }
    if (g->smem_optin < size_t(kSmemLaunch)) { *why = "not enough shared memory"; return false; }
    if (!strides_ok(a.q, a.q_strides, a.B, a.Hq, a.Lq, a.D) || !strides_ok(a.k, a.k_strides, a.B, a.Hkv, a.Lk, a.D) ||
        !strides_ok(a.v, a.v_strides, a.B, a.Hkv, a.Lk, a.D) || !strides_ok(a.out, a.o_strides, a.B, a.Hq, a.Lq, a.D)) {
        *why = "pointers or strides are not 16-byte aligned";
        return false;
    }
    return true;
}

int sdpa_tc_launch(Gpu* g, const paras_sdpa_args& a, float scale, cudaStream_t s, const RopeTables* rope,
                   const char** variant) {
    int st = check_status_word(g);  // an earlier launch's failure is reported once, here
    if (st != PARAS_OK) return st;
    const SplitPlan sp = split_plan(g, a, rope != nullptr);
    if (variant)
        *variant = rope ? "tcgen05_rope" : sp.pack_shift ? (sp.nsplit > 1 ? "tcgen05_packed_split" : "tcgen05_packed")
                                                         : (sp.nsplit > 1 ? "tcgen05_split" : "tcgen05");
    void* scratch = nullptr;
    bool own = false;
    if (sp.nsplit > 1) {
        if (a.workspace) {
            if (a.workspace_bytes < sp.bytes)
                return fail(PARAS_E_INVALID, "paras sdpa: workspace of %zu bytes is smaller than %zu", a.workspace_bytes, sp.bytes);
            if (reinterpret_cast<uintptr_t>(a.workspace) & 15u)
                return fail(PARAS_E_INVALID, "paras sdpa: workspace must be 16-byte aligned");
            scratch = a.workspace;
        } else {
            if ((st = paras_b200_malloc_async(a.gpu, sp.bytes, s, &scratch)) != PARAS_OK) return st;
            own = true;
        }
    }
    void* lens = nullptr;   // kv_len and key_prefix of a key-padding mask
    bool gate_pair = false;  // launch the causal kernel and the masked kernel, the device picks by the mask check
    const int* lens_gate = nullptr;   // likewise with the LENS kernel first (key counts per batch element), gated on this flag
    bool lens_causal = false;
    auto release = [&](int status) {
        if (lens) {
            const int st3 = paras_b200_free_async(a.gpu, lens, s);
            if (status == PARAS_OK) status = st3;
        }
        if (!own) return status;
        const int st2 = paras_b200_free_async(a.gpu, scratch, s);
        return status != PARAS_OK ? status : st2;
    };
    CUtensorMap mq, mk, mv, mo;
    if (sp.pack_shift) st = make_map(&mq, a.q, a.dtype, a.B, a.Hq, a.Lq, a.D, a.q_strides, 1 << sp.pack_shift, BM >> sp.pack_shift);
    else st = make_map(&mq, a.q, a.dtype, a.B, a.Hq, a.Lq, a.D, a.q_strides);
    if (st != PARAS_OK) return release(st);
    if ((st = make_map(&mk, a.k, a.dtype, a.B, a.Hkv, a.Lk, a.D, a.k_strides)) != PARAS_OK) return release(st);
    if ((st = make_map(&mv, a.v, a.dtype, a.B, a.Hkv, a.Lk, a.D, a.v_strides)) != PARAS_OK) return release(st);
    if (sp.nsplit > 1) {
        const int rows = sp.nsplit * sp.lq_pad;
        const int64_t pst[3] = {int64_t(a.Hq) * rows * a.D, int64_t(rows) * a.D, a.D};
        st = make_map(&mo, scratch, a.dtype, a.B, a.Hq, rows, a.D, pst, 32);
    } else {
        st = make_map(&mo, a.out, a.dtype, a.B, a.Hq, a.Lq, a.D, a.o_strides, 32);
    }
    if (st != PARAS_OK) return release(st);
    TcParams p{};
    p.out = a.out;
    p.lse = a.lse;
    p.nsplit = sp.nsplit;
    p.split_tiles = sp.split_tiles;
    p.lq_pad = sp.lq_pad;
    p.pack_shift = sp.pack_shift;
    p.lse_bh = a.Lq;
    if (sp.nsplit > 1) {
        p.lse = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + sp.o_bytes);
        p.lse_bh = int64_t(sp.nsplit) * sp.lq_pad;
    }
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk;
    for (int i = 0; i < 3; ++i) p.os[i] = a.o_strides[i];
    p.causal = a.causal;
    p.scale = scale;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.inv_scale_log2 = 1.0f / p.scale_log2;
    p.inv_scale = 1.0f / scale;
    p.mask = a.mask;
    p.mask_kind = a.mask ? a.mask_kind : 0;
    for (int i = 0; i < 4; ++i) p.ms[i] = a.mask_strides[i];
    // a dimension of extent 1 is never stepped along: its stride reads as 0, like a broadcast one
    if (a.B == 1) p.ms[0] = 0;
    if (a.Hq == 1) p.ms[1] = 0;
    if (a.Lq == 1) p.ms[2] = 0;
    // -60000 (fp16's most negative values) times scale * log2(e) must be far below the -149 at which exp2 gives 0
    const float masked_below = scale * 1.4426950408889634f * 60000.0f > 1000.0f ? -60000.0f : -INFINITY;
    if (p.mask_kind && p.ms[1] == 0 && p.ms[2] == 0 && p.ms[3] == 1 && a.Lk > 1) {
        if ((st = paras_b200_malloc_async(a.gpu, size_t(2 * a.B + 1) * sizeof(int), s, &lens)) != PARAS_OK) return release(st);
        int* li = static_cast<int*>(lens);
        if (cudaMemsetAsync(li + 2 * a.B, 1, sizeof(int), s) != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: memset failed"));
        key_mask_scan_kernel<<<unsigned(a.B), 256, 0, s>>>(a.mask, p.ms[0], a.Lk, p.mask_kind, a.dtype == PARAS_BF16 ? 1 : 0,
                                                          masked_below, li, li + a.B, li + 2 * a.B);
        lens_gate = li + 2 * a.B;   // every batch element's valid keys are a prefix: the kernel without mask code does
        if (cudaGetLastError() != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: mask scan launch failed"));
        p.kv_len = li;
        p.key_prefix = li + a.B;
    } else if (p.mask_kind && p.ms[0] == 0 && p.ms[1] == 0 && p.ms[3] == 1 && a.Lq > 1 && a.Lk > 1) {
        // one [Lq, Lk] mask for every batch element and head: is it the causal mask written out?
        if ((st = paras_b200_malloc_async(a.gpu, sizeof(int), s, &lens)) != PARAS_OK) return release(st);
        int* flag = static_cast<int*>(lens);
        if (cudaMemsetAsync(flag, 1, sizeof(int), s) != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: memset failed"));
        const int64_t spans = int64_t(a.Lq) * ((a.Lk + 15) / 16);
        const int sms_ = g->sm_count > 0 ? g->sm_count : 148;
        const unsigned blocks = unsigned(std::min<int64_t>((spans + 255) / 256, int64_t(sms_) * 8));
        causal_check_kernel<<<blocks, 256, 0, s>>>(a.mask, 0, p.ms[2], a.Lq, a.Lk, p.mask_kind, a.dtype == PARAS_BF16 ? 1 : 0,
                                                   masked_below, nullptr, flag);
        if (cudaGetLastError() != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: mask check launch failed"));
        p.mask_is_causal = flag;
        gate_pair = a.D == 128 || a.D == 64;
    } else if (p.mask_kind && p.ms[0] != 0 && p.ms[1] == 0 && p.ms[2] != 0 && p.ms[3] == 1 && a.Lq > 1 && a.Lk > 1) {
        // one [Lq, Lk] mask per batch element, shared by its heads: causal over right-padded sequences?
        if ((st = paras_b200_malloc_async(a.gpu, size_t(a.B + 1) * sizeof(int), s, &lens)) != PARAS_OK) return release(st);
        int* li = static_cast<int*>(lens);
        if (cudaMemsetAsync(li + a.B, 1, sizeof(int), s) != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: memset failed"));
        const int64_t spans = int64_t(a.Lq) * ((a.Lk + 15) / 16);
        const int sms_ = g->sm_count > 0 ? g->sm_count : 148;
        const unsigned chunks = unsigned(std::max<int64_t>(1, std::min<int64_t>((spans + 255) / 256, int64_t(sms_) * 8 / a.B)));
        causal_check_kernel<<<dim3(chunks, unsigned(a.B)), 256, 0, s>>>(a.mask, p.ms[0], p.ms[2], a.Lq, a.Lk, p.mask_kind,
                                                                      a.dtype == PARAS_BF16 ? 1 : 0, masked_below, li, li + a.B);
        if (cudaGetLastError() != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: mask check launch failed"));
        p.kv_len = li;
        p.kv_len_if_causal = 1;
        p.mask_is_causal = li + a.B;
        lens_gate = li + a.B;
        lens_causal = true;
    }
    p.status = g->status_dev;
    if (rope) {
        if (a.D != 128 || p.mask_kind)
            return fail(PARAS_E_UNSUPPORTED, "paras sdpa: the rotary prologue takes head dim 128 and no mask tensor");
        p.rope_cos = rope->cos; p.rope_sin = rope->sin; p.rope_pos0 = rope->pos0;
    }
    p.nq = (a.Lq + kTilesPerCta * BM - 1) / (kTilesPerCta * BM);
    p.npair = (p.nq + 1) / 2;
    const int64_t per_split = sp.pack_shift ? int64_t(a.B) * a.Hkv : int64_t(a.B) * a.Hq * p.npair;
    p.split_units = int(std::min<int64_t>(per_split, INT32_MAX));
    const int64_t units = per_split * p.nsplit;
    if (units > INT32_MAX) return release(fail(PARAS_E_UNSUPPORTED, "paras sdpa: too many work units"));
    p.units = int(units);
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    dim3 grid(unsigned(units < sms ? units : sms));  // persistent: one CTA per SM
    auto launch = [&](auto kernel) -> int {
        PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLaunch));
        kernel<<<grid, kThreads, kSmemLaunch, s>>>(mq, mk, mv, mo, p);
        return PARAS_OK;
    };
    const bool bf = a.dtype == PARAS_BF16;
    if (sp.pack_shift && sp.nsplit > 1) {
        if (a.D == 128) st = bf ? launch(sdpa_tc_kernel<true, false, 128, false, true, true>) : launch(sdpa_tc_kernel<false, false, 128, false, true, true>);
        else st = bf ? launch(sdpa_tc_kernel<true, false, 64, false, true, true>) : launch(sdpa_tc_kernel<false, false, 64, false, true, true>);
    } else if (sp.pack_shift) {
        if (a.D == 128) st = bf ? launch(sdpa_tc_kernel<true, false, 128, false, false, true>) : launch(sdpa_tc_kernel<false, false, 128, false, false, true>);
        else st = bf ? launch(sdpa_tc_kernel<true, false, 64, false, false, true>) : launch(sdpa_tc_kernel<false, false, 64, false, false, true>);
    } else if (sp.nsplit > 1) {
        if (a.D == 128) st = bf ? launch(sdpa_tc_kernel<true, false, 128, false, true>) : launch(sdpa_tc_kernel<false, false, 128, false, true>);
        else st = bf ? launch(sdpa_tc_kernel<true, false, 64, false, true>) : launch(sdpa_tc_kernel<false, false, 64, false, true>);
    } else if (rope) {
        st = bf ? launch(sdpa_tc_kernel<true, false, 128, true>) : launch(sdpa_tc_kernel<false, false, 128, true>);
    } else {
        if (p.mask_kind && lens_gate) {
            const TcParams keep = p;
            p.mask = nullptr; p.mask_kind = 0; p.causal = lens_causal ? 1 : 0;
            p.key_prefix = nullptr; p.mask_is_causal = nullptr; p.kv_len_if_causal = 0;
            p.gate = lens_gate; p.gate_want = 1;
            if (a.D == 128) st = bf ? launch(sdpa_tc_kernel<true, false, 128, false, false, false, true>) : launch(sdpa_tc_kernel<false, false, 128, false, false, false, true>);
            else st = bf ? launch(sdpa_tc_kernel<true, false, 64, false, false, false, true>) : launch(sdpa_tc_kernel<false, false, 64, false, false, false, true>);
            p = keep;
            p.gate = lens_gate; p.gate_want = 0;
            if (st != PARAS_OK) return release(st);
        } else if (p.mask_kind && gate_pair) {
            // The mask may be the causal mask: the causal kernel is launched for that case (it is a tenth faster
            // than the masked kernel running without its mask) and returns at once otherwise; the masked kernel
            // that follows does the opposite.
            const TcParams keep = p;
            p.mask = nullptr; p.mask_kind = 0; p.causal = 1;
            p.gate = keep.mask_is_causal; p.gate_want = 1; p.mask_is_causal = nullptr;
            if (a.D == 128) st = bf ? launch(sdpa_tc_kernel<true, false, 128>) : launch(sdpa_tc_kernel<false, false, 128>);
            else st = bf ? launch(sdpa_tc_kernel<true, false, 64>) : launch(sdpa_tc_kernel<false, false, 64>);
            p = keep;
            p.gate = keep.mask_is_causal; p.gate_want = 0; p.mask_is_causal = nullptr;
            if (st != PARAS_OK) return release(st);
        }
        if (a.D == 128) {
            if (p.mask_kind) st = bf ? launch(sdpa_tc_kernel<true, true, 128>) : launch(sdpa_tc_kernel<false, true, 128>);
            else st = bf ? launch(sdpa_tc_kernel<true, false, 128>) : launch(sdpa_tc_kernel<false, false, 128>);
        } else {
            if (p.mask_kind) st = bf ? launch(sdpa_tc_kernel<true, true, 64>) : launch(sdpa_tc_kernel<false, true, 64>);
            else st = bf ? launch(sdpa_tc_kernel<true, false, 64>) : launch(sdpa_tc_kernel<false, false, 64>);
        }
    }
    if (st != PARAS_OK) return release(st);
    if (cudaGetLastError() != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: sdpa_tc_kernel launch failed"));
    if (sp.nsplit > 1) {
        CombineParams c{};
        c.part_o = static_cast<const uint16_t*>(scratch);
        c.part_lse = p.lse;
        c.out = a.out;
        c.lse = a.lse;
        c.B = a.B; c.Hq = a.Hq; c.Lq = a.Lq; c.Lk = a.Lk; c.causal = a.causal;
        c.nsplit = sp.nsplit; c.split_tiles = sp.split_tiles; c.lq_pad = sp.lq_pad;
        for (int i = 0; i < 3; ++i) c.os[i] = a.o_strides[i];
        const int64_t threads = int64_t(a.B) * a.Hq * a.Lq * (a.D / 8);
        const unsigned blocks = unsigned((threads + 255) / 256);
        if (a.D == 128) {
            if (bf) sdpa_tc_combine_kernel<true, 128><<<blocks, 256, 0, s>>>(c);
            else sdpa_tc_combine_kernel<false, 128><<<blocks, 256, 0, s>>>(c);
        } else {
            if (bf) sdpa_tc_combine_kernel<true, 64><<<blocks, 256, 0, s>>>(c);
            else sdpa_tc_combine_kernel<false, 64><<<blocks, 256, 0, s>>>(c);
        }
        if (cudaGetLastError() != cudaSuccess) return release(fail(PARAS_E_CUDA, "paras sdpa: combine launch failed"));
    }
    return release(PARAS_OK);
}

}  // namespace pb
