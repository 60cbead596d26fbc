// Attention with its weights made explicit: dropout on the weights, a caller's dropout mask, and
// the weights tensor itself -- the parts of the reference's sdpa_math (csrc/ops/attention_ops.cpp:
// 128-135) that need every normalised weight, which a flash kernel never forms.
//
// One warp per query row, two passes over the row's keys on CUDA cores: the first finds the row's
// max and sum (online), the second recomputes each score, normalises it, rounds it to the tensors'
// dtype (the reference's softmax output, csrc/ops/pointwise_ops.cpp:926-981), applies dropout,
// optionally stores the weight, and accumulates weight * V in fp32 -- so the product uses exactly
// the rounded weights the reference's matmul sees.  Dropout follows the reference bit for bit:
//   native_dropout (csrc/ops/random_ops.cpp:140-176): weight i of the contiguous [B,Hq,Lq,Lk]
//     tensor is kept when to_float(Philox2x32-10(seed, sequence, i).r0) < float(1 - p) and becomes
//     dtype(float(w) * (1.0f / keep)), else 0;
//   a given dropout_mask: dtype(dtype(w * mask) / (1 - p)).
// This is the opt-in slow path: O(Lq * Lk * D) on CUDA cores, scores computed twice.
#include <cmath>

#include "sdpa_common.cuh"

namespace pb {
namespace {

constexpr int kRowsPerBlock = 4;
constexpr int kMaxD = 256;

struct WeightsParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;
    void* attn_out;
    const void* mask;
    const void* dmask;
    int mask_kind, dmask_kind;
    int B, Hq, Hkv, Lq, Lk, D;
    int64_t qs[3], ks[3], vs[3], os[3], ms[4], ds[4];
    int causal;
    float scale;
    float keep;       // float(1 - p)
    float inv_keep;   // 1.0f / keep
    float one_minus_p_scalar;   // (1 - p) as the reference's scalar operand, rounded to the dtype
    int dropout;      // 0 none, 1 Philox, 2 given mask
    uint64_t seed, sequence;
};

template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
sdpa_weights_kernel(const WeightsParams p) {
    __shared__ float sq[kRowsPerBlock][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qi = blockIdx.x * kRowsPerBlock + warp;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int D = p.D;
    if (qi >= p.Lq) return;

    const T* qrow = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + int64_t(qi) * p.qs[2];
    for (int d = lane; d < D; d += 32) sq[warp][d] = to_f32<T>(qrow[d]);
    __syncwarp();
    const int k_end = p.causal ? min(p.Lk, qi + 1) : p.Lk;   // top-left aligned: keys 0..qi
    const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
    const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];

    // the scaled, masked score of `key` for this row (-inf when masked out)
    auto score = [&](int key) -> float {
        const T* krow = kbase + int64_t(key) * p.ks[2];
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(sq[warp][d], to_f32<T>(krow[d]), dot);
        float s = dot * p.scale;
        if (p.mask_kind) {
            const int64_t mo = b * p.ms[0] + h * p.ms[1] + int64_t(qi) * p.ms[2] + int64_t(key) * p.ms[3];
            if (p.mask_kind == 1) {
                if (!static_cast<const unsigned char*>(p.mask)[mo]) s = -INFINITY;
            } else if (p.mask_kind == 2) {
                s += to_f32<T>(static_cast<const T*>(p.mask)[mo]);
            } else {
                s += static_cast<const float*>(p.mask)[mo];
            }
        }
        return s;
    };

    // pass 1: row max and sum
    float m = -INFINITY, l = 0.f;
    for (int k0 = 0; k0 < k_end; k0 += 32) {
        const int key = k0 + lane;
        const float s = key < k_end ? score(key) : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        float pj = 0.f, alpha = 1.f;
        if (m_new != -INFINITY) {
            pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        }
        l = l * alpha + warp_sum(pj);
        m = m_new;
    }

    // pass 2: the weights themselves
    float acc[kMaxD / 32];
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) acc[i] = 0.f;
    const int64_t row = (int64_t(b) * p.Hq + h) * p.Lq + qi;
    T* wrow = p.attn_out ? static_cast<T*>(p.attn_out) + row * p.Lk : nullptr;
    const float inv = 1.0f / l;   // l == 0: every key masked out -> 0 * inf = NaN weights, as in the reference
    for (int k0 = 0; k0 < p.Lk; k0 += 32) {
        const int key = k0 + lane;
        float w = 0.f;   // keys the causal mask hides have weight exp(-inf) = 0
        if (key < p.Lk) {
            if (key < k_end) {
                const float s = score(key);
                w = round_to<T>((s == -INFINITY && m != -INFINITY) ? 0.f : expf(s - m) * inv);
            } else if (l == 0.f) {
                w = __int_as_float(0x7fc00000);
            }
            if (p.dropout == 1) {
                const uint64_t idx = uint64_t(row) * uint64_t(p.Lk) + uint64_t(key);
                const float u = float(philox2x32_r0(p.seed, p.sequence, idx) >> 8) * (1.0f / 16777216.0f);
                w = u < p.keep ? round_to<T>(w * p.inv_keep) : 0.f;
            } else if (p.dropout == 2) {
                const int64_t mo = b * p.ds[0] + h * p.ds[1] + int64_t(qi) * p.ds[2] + int64_t(key) * p.ds[3];
                float mv;
                if (p.dmask_kind == 1) mv = static_cast<const unsigned char*>(p.dmask)[mo] ? 1.f : 0.f;
                else if (p.dmask_kind == 2) mv = to_f32<T>(static_cast<const T*>(p.dmask)[mo]);
                else mv = static_cast<const float*>(p.dmask)[mo];
                w = round_to<T>(round_to<T>(w * mv) / p.one_minus_p_scalar);
            }
            if (wrow) wrow[key] = from_f32<T>(w);
        }
        const int valid = min(32, p.Lk - k0);
        for (int j = 0; j < valid; ++j) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (wj == 0.f) continue;   // uniform across the warp
            const T* vrow = vbase + int64_t(k0 + j) * p.vs[2];
#pragma unroll
            for (int i = 0; i < kMaxD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(wj, to_f32<T>(vrow[d]), acc[i]);
            }
        }
    }
    T* orow = static_cast<T*>(p.out) + b * p.os[0] + h * p.os[1] + int64_t(qi) * p.os[2];
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = from_f32<T>(acc[i]);
    }
    if (p.lse && lane == 0) p.lse[row] = (l == 0.f) ? -INFINITY : m + logf(l);
}

}  // namespace

bool sdpa_wants_weights(const paras_sdpa_args& a) {
    return a.dropout_p > 0.0 || a.dropout_mask != nullptr || a.attn_out != nullptr;
}

int sdpa_weights_launch(Gpu* g, const paras_sdpa_args& a, float scale, cudaStream_t s) {
    (void)g;
    if (a.D > kMaxD)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: head dim %d exceeds kernel limit %d", a.D, kMaxD);
    if (a.B > 65535 || a.Hq > 65535)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: batch or heads exceed the grid limit");
    if (!(a.dropout_p >= 0.0) || a.dropout_p >= 1.0)
        return fail(PARAS_E_INVALID, "paras sdpa: dropout_p must be in [0, 1), got %g", a.dropout_p);
    if (a.dropout_mask && (a.dropout_mask_kind < 1 || a.dropout_mask_kind > 3))
        return fail(PARAS_E_INVALID, "paras sdpa: bad dropout mask kind %d", a.dropout_mask_kind);
    WeightsParams p{};
    p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out; p.lse = a.lse; p.attn_out = a.attn_out;
    p.mask = a.mask; p.mask_kind = a.mask ? a.mask_kind : 0;
    p.dmask = a.dropout_mask; p.dmask_kind = a.dropout_mask_kind;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk; p.D = a.D;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = a.q_strides[i]; p.ks[i] = a.k_strides[i]; p.vs[i] = a.v_strides[i]; p.os[i] = a.o_strides[i];
    }
    for (int i = 0; i < 4; ++i) { p.ms[i] = a.mask_strides[i]; p.ds[i] = a.dropout_mask_strides[i]; }
    p.causal = a.causal;
    p.scale = scale;
    p.keep = float(1.0 - a.dropout_p);
    p.inv_keep = 1.0f / p.keep;
    float omp = float(1.0 - a.dropout_p);   // the divisor is wrapped into a 0-dim tensor of the dtype
    if (a.dtype == PARAS_BF16) omp = __bfloat162float(__float2bfloat16_rn(omp));
    else if (a.dtype == PARAS_F16) omp = __half2float(__float2half_rn(omp));
    p.one_minus_p_scalar = omp;
    p.dropout = a.dropout_p > 0.0 ? (a.dropout_mask ? 2 : 1) : 0;
    p.seed = a.rng_seed; p.sequence = a.rng_sequence;
    dim3 grid((a.Lq + kRowsPerBlock - 1) / kRowsPerBlock, a.Hq, a.B);
    switch (a.dtype) {
        case PARAS_F32: sdpa_weights_kernel<float><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
        case PARAS_BF16: sdpa_weights_kernel<__nv_bfloat16><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
        default: sdpa_weights_kernel<__half><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
    }
    PB_LAUNCH_CHECK("sdpa_weights_kernel");
    return PARAS_OK;
}

}  // namespace pb
