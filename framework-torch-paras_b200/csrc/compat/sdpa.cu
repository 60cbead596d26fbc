// paras_b200_sdpa_fwd: argument validation and kernel selection.
//
// Mirrors the checks of the reference's sdpa_math (csrc/ops/attention_ops.cpp:77-98):
// heads must divide for GQA, is_causal and a mask tensor are exclusive, the default scale
// is 1/sqrt(D).  Selection:
//   * 16-bit, D == 128, no mask tensor, long queries  -> tcgen05/TMEM/TMA kernel
//   * 16-bit, D == 128, no mask tensor, few queries   -> tensor-core split-KV decode kernel
//   * everything else                                  -> CUDA-core kernel (sdpa_simt.cu)
// There is no host fallback: an unsupported request is an error.
#include <cmath>

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

int paras_b200_sdpa_workspace_bytes(const paras_sdpa_args* a, size_t* bytes) {
    if (!bytes) return fail(PARAS_E_INVALID, "paras sdpa: null output");
    *bytes = 0;
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    const char* why;
    const int64_t rows = int64_t(a->B) * a->Hq * a->Lq;
    switch (pb::choose(g, *a, &why)) {
        case pb::Path::Tensor: break;
        case pb::Path::Decode:
            *bytes = pb::split_workspace_bytes(rows, a->D, pb::sdpa_decode_pick_splits(g, *a));
            break;
        case pb::Path::Simt:
            *bytes = pb::split_workspace_bytes(rows, a->D, pb::sdpa_simt_pick_splits(g, *a));
            break;
    }
    return PARAS_OK;
}

int paras_b200_sdpa_fwd(const paras_sdpa_args* a) {
    int st = pb::validate(a);
    if (st != PARAS_OK) return st;
    Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0) return PARAS_OK;  // empty output
    if (!a->q || !a->out) return fail(PARAS_E_INVALID, "paras sdpa: null pointer");
    if (a->Lk > 0 && (!a->k || !a->v)) return fail(PARAS_E_INVALID, "paras sdpa: null pointer");
    cudaStream_t s = pb::pick_stream(g, a->stream);
    const float scale = pb::effective_scale(*a);
    const char* why = "";
    const pb::Path path = pb::choose(g, *a, &why);
    if ((a->flags & PARAS_SDPA_FORCE_TENSOR) && path == pb::Path::Simt)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: tensor-core kernel unavailable: %s", why);

    if (path == pb::Path::Tensor) {
        st = pb::sdpa_tc_launch(g, *a, scale, s);
        if (st == PARAS_OK) pb::set_last_kernel("tcgen05");
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

}  // extern "C"
