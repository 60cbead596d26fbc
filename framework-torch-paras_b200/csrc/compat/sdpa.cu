// paras_b200_sdpa_fwd: argument validation and kernel selection.
//
// Mirrors the checks of the reference's sdpa_math (csrc/ops/attention_ops.cpp:77-98):
// heads must divide for GQA, is_causal and a mask tensor are exclusive, the default scale
// is 1/sqrt(D).  Selection:
//   * 16-bit, D == 128, no mask tensor, few queries   -> tensor-core split-KV decode kernel
//   * 16-bit, D == 128 or 64 otherwise (masks incl.)  -> tcgen05/TMEM/TMA kernel
//   * everything else                                  -> CUDA-core kernel (sdpa_simt.cu)
//   * dropout, a dropout mask or the weights as output -> two-pass CUDA-core kernel (sdpa_weights.cu)
// There is no host fallback: an unsupported request is an error.
#include <algorithm>
#include <cmath>
#include <mutex>

#include "sdpa_common.cuh"

namespace pb {
namespace {

int validate(const paras_sdpa_args* a) {
    if (!a) return fail(PARAS_E_INVALID, "paras sdpa: null argument block");
    if (a->dtype != PARAS_F32 && a->dtype != PARAS_BF16 && a->dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: unsupported dtype %d", a->dtype);
    if (a->B < 0 || a->Hq < 0 || a->Hkv < 0 || a->Lq < 0 || a->Lk < 0 || a->D < 0)
        return fail(PARAS_E_INVALID, "paras sdpa: negative dimension");
    if (a->Hkv == 0 ? a->Hq != 0 : (a->Hq % a->Hkv) != 0)
        return fail(PARAS_E_INVALID,
                    "paras sdpa: query heads must be a multiple of key/value heads for enable_gqa");
    if (a->causal && a->mask)
        return fail(PARAS_E_INVALID, "paras sdpa: is_causal and attn_mask are mutually exclusive");
    if (a->mask && (a->mask_kind < 1 || a->mask_kind > 3))
        return fail(PARAS_E_INVALID, "paras sdpa: bad mask kind %d", a->mask_kind);
    return PARAS_OK;
}

}  // namespace

float effective_scale(const paras_sdpa_args& a) {
    double sc = a.scale;
    if (a.flags & PARAS_SDPA_REF_SCALE) {
        // the reference multiplies by a 0-dim tensor of the scores' dtype
        float f = float(sc);
        if (a.dtype == PARAS_BF16) f = __bfloat162float(__float2bfloat16_rn(f));
        else if (a.dtype == PARAS_F16) f = __half2float(__float2half_rn(f));
        sc = f;
    }
    return float(sc);
}

namespace {

enum class Path { Tensor, Decode, Simt };

Path choose(const Gpu* g, const paras_sdpa_args& a, const char** why) {
    *why = "";
    if (a.flags & PARAS_SDPA_FORCE_SIMT) return Path::Simt;
    const char* why_tc = "";
    const char* why_dec = "";
    const bool tc = sdpa_tc_supported(g, a, &why_tc);
    const bool dec = sdpa_decode_supported(g, a, &why_dec);
    if (a.flags & PARAS_SDPA_FORCE_TENSOR) {
        if (tc) return Path::Tensor;
        if (dec) return Path::Decode;
        *why = why_tc;
        return Path::Simt;
    }
    if (dec) return Path::Decode;  // only claims short-query problems
    if (tc) return Path::Tensor;
    *why = why_tc;
    return Path::Simt;
}

}  // namespace
}  // namespace pb

using pb::fail;
using pb::Gpu;

extern "C" {

int paras_b200_sdpa_split_layout(int64_t rows, int32_t D, int32_t splits, size_t* ml_offset,
                                 size_t* o_offset, size_t* bytes) {
    if (rows < 0 || D < 0 || splits < 1) return fail(PARAS_E_INVALID, "paras sdpa: bad split layout request");
    // carve an imaginary scratch at a 16-byte aligned address and report the distances from it
    const uintptr_t base = 1u << 20;
    const pb::SplitWorkspace w = pb::carve_workspace(reinterpret_cast<void*>(base), rows, D, splits);
    if (ml_offset) *ml_offset = splits > 1 ? reinterpret_cast<uintptr_t>(w.ml_part) - base : 0;
    if (o_offset) *o_offset = splits > 1 ? reinterpret_cast<uintptr_t>(w.o_part) - base : 0;
    if (bytes) *bytes = pb::split_workspace_bytes(rows, D, splits);
    return PARAS_OK;
}

int paras_b200_sdpa_workspace_bytes(const paras_sdpa_args* a, size_t* bytes) {
    if (!bytes) return fail(PARAS_E_INVALID, "paras sdpa: null output");
    *bytes = 0;
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    const char* why;
    const int64_t rows = int64_t(a->B) * a->Hq * a->Lq;
    if (pb::sdpa_wants_weights(*a)) return PARAS_OK;   // the two-pass kernel needs no scratch
    switch (pb::choose(g, *a, &why)) {
        case pb::Path::Tensor: *bytes = pb::sdpa_tc_workspace_bytes(g, *a); break;
        case pb::Path::Decode:
            *bytes = pb::split_workspace_bytes(rows, a->D, pb::sdpa_decode_pick_splits(g, *a));
            break;
        case pb::Path::Simt:
            *bytes = pb::split_workspace_bytes(rows, a->D, pb::sdpa_simt_pick_splits(g, *a));
            break;
    }
    return PARAS_OK;
}

int paras_b200_sdpa_mask_is_causal(int gpu, const void* mask, int mask_kind, int dtype, int64_t row_stride, int32_t Lq,
                                   int32_t Lk, double scale, void* stream, int* result) {
    if (!result) return fail(PARAS_E_INVALID, "paras sdpa: null output");
    *result = 0;
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    return pb::sdpa_mask_is_causal(g, gpu, mask, mask_kind, dtype, row_stride, Lq, Lk, float(scale), pb::pick_stream(g, stream), result);
}

int paras_b200_sdpa_fwd(const paras_sdpa_args* a) {
    pb::NvtxRange range("paras_b200_sdpa_fwd");
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0) return PARAS_OK;  // empty output
    if (!a->q || !a->out) return fail(PARAS_E_INVALID, "paras sdpa: null pointer");
    if (a->Lk > 0 && (!a->k || !a->v)) return fail(PARAS_E_INVALID, "paras sdpa: null pointer");
    cudaStream_t s = pb::pick_stream(g, a->stream);
    const float scale = pb::effective_scale(*a);
    if (pb::sdpa_wants_weights(*a)) {
        if (a->flags & PARAS_SDPA_FORCE_TENSOR)
            return fail(PARAS_E_UNSUPPORTED, "paras sdpa: dropout and the weights output run on CUDA cores only");
        if (a->Lk == 0) return fail(PARAS_E_UNSUPPORTED, "paras sdpa: dropout / weights output with no keys");
        st = pb::sdpa_weights_launch(g, *a, scale, s);
        if (st == PARAS_OK) pb::set_last_kernel("weights");
        return st;
    }
    const char* why = "";
    const pb::Path path = pb::choose(g, *a, &why);
    if ((a->flags & PARAS_SDPA_FORCE_TENSOR) && path == pb::Path::Simt)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: tensor-core kernel unavailable: %s", why);

    if (path == pb::Path::Tensor) {
        const char* variant = "tcgen05";
        st = pb::sdpa_tc_launch(g, *a, scale, s, nullptr, &variant);
        if (st == PARAS_OK) pb::set_last_kernel(variant);
        return st;
    }

    const int64_t rows = int64_t(a->B) * a->Hq * a->Lq;
    const int splits = path == pb::Path::Decode ? pb::sdpa_decode_pick_splits(g, *a)
                                                : pb::sdpa_simt_pick_splits(g, *a);
    const size_t need = pb::split_workspace_bytes(rows, a->D, splits);
    void* wsmem = nullptr;
    bool own = false;
    if (need) {
        if (a->workspace) {
            if (a->workspace_bytes < need)
                return fail(PARAS_E_INVALID, "paras sdpa: workspace of %zu bytes is smaller than %zu",
                            a->workspace_bytes, need);
            if (reinterpret_cast<uintptr_t>(a->workspace) & 15u)
                return fail(PARAS_E_INVALID, "paras sdpa: workspace must be 16-byte aligned");
            wsmem = a->workspace;
        } else {
            st = paras_b200_malloc_async(a->gpu, need, s, &wsmem);
            if (st != PARAS_OK) return st;
            own = true;
        }
    }
    const pb::SplitWorkspace ws = pb::carve_workspace(wsmem, rows, a->D, splits);
    if (path == pb::Path::Decode) {
        st = pb::sdpa_decode_launch(g, *a, scale, ws, s);
        if (st == PARAS_OK) pb::set_last_kernel("decode_mma");
    } else {
        st = pb::sdpa_simt_launch(g, *a, scale, ws, s);
        if (st == PARAS_OK) pb::set_last_kernel(splits > 1 ? "simt_splitkv" : "simt");
    }
    if (own) {
        const int st2 = paras_b200_free_async(a->gpu, wsmem, s);
        if (st == PARAS_OK) st = st2;
    }
    return st;
}

// ---- attention with the rotary embedding in its prologue -------------------------------------
int paras_b200_sdpa_rope_fwd(const paras_sdpa_args* a, const void* cosv, const void* sinv, int64_t table_rows,
                             int64_t q_pos0) {
    pb::NvtxRange range("paras_b200_sdpa_rope_fwd");
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    if (a->mask || pb::sdpa_wants_weights(*a))
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa_rope: no mask tensor, dropout or weights output");
    if (a->D % 2) return fail(PARAS_E_INVALID, "paras sdpa_rope: head dim must be even");
    if (q_pos0 < 0 || q_pos0 + a->Lq > table_rows || a->Lk > table_rows)
        return fail(PARAS_E_INVALID, "paras sdpa_rope: cos / sin tables of %lld rows do not cover the positions",
                    (long long)table_rows);
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0) return PARAS_OK;
    if (!a->q || !a->out || !cosv || !sinv || (a->Lk > 0 && (!a->k || !a->v)))
        return fail(PARAS_E_INVALID, "paras sdpa_rope: null pointer");
    if (a->Lk == 0) return paras_b200_sdpa_fwd(a);   // nothing to rotate against
    cudaStream_t s = pb::pick_stream(g, a->stream);
    const size_t es = pb::dtype_size(a->dtype);
    const size_t k_bytes = (size_t(a->B) * a->Hkv * a->Lk * a->D * es + 255) & ~size_t(255);
    const size_t q_bytes = (size_t(a->B) * a->Hq * a->Lq * a->D * es + 255) & ~size_t(255);

    // Q is rotated inside the tensor-core kernel when that kernel runs (and its tables can be read
    // 16 bytes at a time); otherwise by the same streaming pass as K.
    paras_sdpa_args sub = *a;
    sub.stream = s;
    const char* why = "";
    const bool q_in_kernel = pb::choose(g, sub, &why) == pb::Path::Tensor && a->D == 128 &&
                             ((reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv)) & 15u) == 0;
    void* scratch = nullptr;
    st = paras_b200_malloc_async(a->gpu, k_bytes + (q_in_kernel ? 0 : q_bytes), s, &scratch);
    if (st != PARAS_OK) return st;
    char* k_rot = static_cast<char*>(scratch);
    char* q_rot = k_rot + k_bytes;
    // K: every query block reads every key tile it sees, so rotating K where it is consumed would
    // repeat the work once per query block; it is rotated once, here, into scratch.
    st = paras_b200_rope(a->gpu, a->k, a->k_strides, cosv, sinv, k_rot, a->B, a->Hkv, a->Lk, a->D, 0, a->dtype, s);
    sub.k = k_rot;
    sub.k_strides[0] = int64_t(a->Hkv) * a->Lk * a->D;
    sub.k_strides[1] = int64_t(a->Lk) * a->D;
    sub.k_strides[2] = a->D;
    if (st == PARAS_OK && !q_in_kernel) {
        st = paras_b200_rope(a->gpu, a->q, a->q_strides, cosv, sinv, q_rot, a->B, a->Hq, a->Lq, a->D, q_pos0, a->dtype, s);
        sub.q = q_rot;
        sub.q_strides[0] = int64_t(a->Hq) * a->Lq * a->D;
        sub.q_strides[1] = int64_t(a->Lq) * a->D;
        sub.q_strides[2] = a->D;
    }
    if (st == PARAS_OK) {
        if (q_in_kernel) {
            const pb::RopeTables rope{cosv, sinv, q_pos0};
            st = pb::sdpa_tc_launch(g, sub, pb::effective_scale(sub), s, &rope);
            if (st == PARAS_OK) pb::set_last_kernel("tcgen05_rope");
        } else {
            st = paras_b200_sdpa_fwd(&sub);
        }
    }
    const int st2 = paras_b200_free_async(a->gpu, scratch, s);
    return st != PARAS_OK ? st : st2;
}

// ---- attention on host-resident operands ------------------------------------------------
// Per-GPU streams and events of the pipeline below (created on first use, never destroyed).
namespace pb {
namespace {
constexpr int kHostSlots = 3;
struct HostPipe {
    std::mutex mu;
    bool ready = false;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    cudaEvent_t in_done[kHostSlots], comp_done[kHostSlots], out_done[kHostSlots];
};
HostPipe g_host_pipe[16];
}  // namespace
}  // namespace pb

int paras_b200_sdpa_fwd_host(const paras_sdpa_args* a) {
    pb::NvtxRange range("paras_b200_sdpa_fwd_host");
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    if (a->gpu < 0 || a->gpu >= 16) return fail(PARAS_E_UNSUPPORTED, "paras sdpa (host): GPU ordinal out of range");
    if (a->mask || a->lse || a->workspace || pb::sdpa_wants_weights(*a))
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa (host): mask, lse, workspace, dropout and weights output are not taken here");
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0) return PARAS_OK;
    if (!a->q || !a->out || (a->Lk > 0 && (!a->k || !a->v)))
        return fail(PARAS_E_INVALID, "paras sdpa (host): null pointer");
    // each batch element must be one dense [H, L, D] block, so that it moves in one copy
    auto dense = [&](const int64_t* s, int H, int L) {
        return (L <= 1 || s[2] == a->D) && (H <= 1 || s[1] == int64_t(L) * a->D) &&
               (a->B <= 1 || s[0] >= int64_t(H) * L * a->D);
    };
    if (!dense(a->q_strides, a->Hq, a->Lq) || !dense(a->k_strides, a->Hkv, a->Lk) ||
        !dense(a->v_strides, a->Hkv, a->Lk) || !dense(a->o_strides, a->Hq, a->Lq))
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa (host): every batch element must be a dense [H, L, D] block");

    pb::HostPipe& hp = pb::g_host_pipe[a->gpu];
    std::lock_guard<std::mutex> lk(hp.mu);  // one pipeline per GPU at a time
    if (!hp.ready) {
        PB_CUDA(cudaStreamCreateWithFlags(&hp.h2d, cudaStreamNonBlocking));
        PB_CUDA(cudaStreamCreateWithFlags(&hp.d2h, cudaStreamNonBlocking));
        for (int i = 0; i < pb::kHostSlots; ++i) {
            PB_CUDA(cudaEventCreateWithFlags(&hp.in_done[i], cudaEventDisableTiming));
            PB_CUDA(cudaEventCreateWithFlags(&hp.comp_done[i], cudaEventDisableTiming));
            PB_CUDA(cudaEventCreateWithFlags(&hp.out_done[i], cudaEventDisableTiming));
        }
        hp.ready = true;
    }
    cudaStream_t comp = pb::pick_stream(g, a->stream);
    const size_t es = pb::dtype_size(a->dtype);
    const size_t q_b = size_t(a->Hq) * a->Lq * a->D * es, kv_b = size_t(a->Hkv) * a->Lk * a->D * es;
    // Chunks of about 64 MB of operands (16 MB chunks measured 12 % slower end to end: more
    // launches and events per byte, and short copies in both directions share the link worse).  A chunk is a range of batch elements
    // with all their heads or, when one batch element is larger than that, a range of query
    // heads of one batch element together with the kv heads they share (both are dense blocks).
    const int r = a->Hq / a->Hkv;  // query heads per kv head
    const size_t q_h = size_t(a->Lq) * a->D * es, kv_h = size_t(a->Lk) * a->D * es;  // bytes per head
    const size_t per_b = 2 * q_b + 2 * kv_b;
    const size_t target = size_t(64) << 20;
    int nb = 1, nh = a->Hq;
    if (per_b <= target) {
        nb = int(std::min<size_t>(size_t(a->B), std::max<size_t>(1, target / std::max<size_t>(per_b, 1))));
    } else {
        const size_t per_group = 2 * q_h * r + 2 * kv_h;  // one kv head and its query heads
        nh = r * int(std::max<size_t>(1, target / std::max<size_t>(per_group, 1)));
        nh = std::min(nh, a->Hq);
    }
    auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t q_c = up(q_h * nh * nb), kv_c = up(kv_h * (nh / r) * nb);  // per chunk
    const size_t slot_bytes = 2 * q_c + 2 * kv_c;
    void* block = nullptr;
    st = paras_b200_malloc_async(a->gpu, slot_bytes * pb::kHostSlots, comp, &block);
    if (st != PARAS_OK) return st;
    // the copy streams may touch the block only after the allocation is ordered before them
    cudaEvent_t alloc_ev = hp.comp_done[0];
    cudaError_t ce = cudaEventRecord(alloc_ev, comp);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(hp.h2d, alloc_ev, 0);
    const bool pinned = pb::host_ptr_is_pinned(a->q) && pb::host_ptr_is_pinned(a->k) &&
                        pb::host_ptr_is_pinned(a->v) && pb::host_ptr_is_pinned(a->out);
    int rc = ce == cudaSuccess ? PARAS_OK : fail(PARAS_E_CUDA, "paras sdpa (host): %s", cudaGetErrorString(ce));
    int chunk = 0;
    for (int b0 = 0; rc == PARAS_OK && ce == cudaSuccess && b0 < a->B; b0 += nb) {
        for (int h0 = 0; rc == PARAS_OK && ce == cudaSuccess && h0 < a->Hq; h0 += nh, ++chunk) {
            const int n = std::min(nb, a->B - b0);
            const int hq = std::min(nh, a->Hq - h0), hk = hq / r;
            const int slot = chunk % pb::kHostSlots;
            char* dq = static_cast<char*>(block) + size_t(slot) * slot_bytes;
            char* dk = dq + q_c;
            char* dv = dk + kv_c;
            char* dout = dv + kv_c;
            // the slot is free once the chunk that used it last has been copied out
            if (chunk >= pb::kHostSlots) ce = cudaStreamWaitEvent(hp.h2d, hp.out_done[slot], 0);
            if (ce != cudaSuccess) break;
            // n batch elements x `heads` heads starting at head `first`: one dense block per batch element
            auto h2d = [&](char* dst, const void* src, const int64_t* strides, size_t head_bytes, int first, int heads) {
                const size_t bytes = head_bytes * heads;
                for (int i = 0; i < n && rc == PARAS_OK; ++i) {
                    const char* s0 = static_cast<const char*>(src) + size_t(b0 + i) * size_t(strides[0]) * es +
                                     size_t(first) * head_bytes;
                    // consecutive batch elements that are also consecutive in memory go in one copy
                    if (i == 0 && n > 1 && size_t(strides[0]) * es == bytes) {
                        rc = paras_b200_memcpy_h2d(a->gpu, dst, s0, bytes * n, hp.h2d, 0);
                        break;
                    }
                    rc = paras_b200_memcpy_h2d(a->gpu, dst + i * bytes, s0, bytes, hp.h2d, 0);
                }
            };
            h2d(dq, a->q, a->q_strides, q_h, h0, hq);
            h2d(dk, a->k, a->k_strides, kv_h, h0 / r, hk);
            h2d(dv, a->v, a->v_strides, kv_h, h0 / r, hk);
            if (rc != PARAS_OK) break;
            ce = cudaEventRecord(hp.in_done[slot], hp.h2d);
            if (ce == cudaSuccess) ce = cudaStreamWaitEvent(comp, hp.in_done[slot], 0);
            if (ce != cudaSuccess) break;
            paras_sdpa_args sub = *a;
            sub.q = dq; sub.k = dk; sub.v = dv; sub.out = dout;
            sub.B = n; sub.Hq = hq; sub.Hkv = hk;
            sub.q_strides[0] = sub.o_strides[0] = int64_t(hq) * a->Lq * a->D;
            sub.k_strides[0] = sub.v_strides[0] = int64_t(hk) * a->Lk * a->D;
            sub.q_strides[1] = sub.o_strides[1] = int64_t(a->Lq) * a->D;
            sub.k_strides[1] = sub.v_strides[1] = int64_t(a->Lk) * a->D;
            sub.q_strides[2] = sub.o_strides[2] = sub.k_strides[2] = sub.v_strides[2] = a->D;
            sub.stream = comp;
            rc = paras_b200_sdpa_fwd(&sub);
            if (rc != PARAS_OK) break;
            ce = cudaEventRecord(hp.comp_done[slot], comp);
            if (ce == cudaSuccess) ce = cudaStreamWaitEvent(hp.d2h, hp.comp_done[slot], 0);
            if (ce != cudaSuccess) break;
            const size_t o_bytes = q_h * hq;
            for (int i = 0; i < n && rc == PARAS_OK && ce == cudaSuccess; ++i) {
                char* o0 = static_cast<char*>(a->out) + size_t(b0 + i) * size_t(a->o_strides[0]) * es + size_t(h0) * q_h;
                if (pinned) {
                    if (i == 0 && n > 1 && size_t(a->o_strides[0]) * es == o_bytes) {
                        ce = cudaMemcpyAsync(o0, dout, o_bytes * n, cudaMemcpyDeviceToHost, hp.d2h);
                        break;
                    }
                    ce = cudaMemcpyAsync(o0, dout + i * o_bytes, o_bytes, cudaMemcpyDeviceToHost, hp.d2h);
                } else {
                    // pageable result: the staged copy blocks this thread until the piece is on the host
                    rc = paras_b200_memcpy_d2h(a->gpu, o0, dout + i * o_bytes, o_bytes, hp.d2h);
                }
            }
            if (rc == PARAS_OK && ce == cudaSuccess) ce = cudaEventRecord(hp.out_done[slot], hp.d2h);
        }
    }
    // everything drains before the block goes back to the pool and the caller reads the result
    cudaError_t c1 = cudaStreamSynchronize(hp.h2d);
    cudaError_t c2 = cudaStreamSynchronize(comp);
    cudaError_t c3 = cudaStreamSynchronize(hp.d2h);
    const int st2 = paras_b200_free_async(a->gpu, block, comp);
    if (rc != PARAS_OK) return rc;
    for (cudaError_t e : {ce, c1, c2, c3})
        if (e != cudaSuccess) return fail(PARAS_E_CUDA, "paras sdpa (host): %s", cudaGetErrorString(e));
    if (st2 != PARAS_OK) return st2;
    return pb::check_status_word(g);
}

}  // extern "C"
