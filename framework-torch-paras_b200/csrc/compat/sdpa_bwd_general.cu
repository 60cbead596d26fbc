// Attention gradients for everything the fused backward does not take: an explicit attn_mask,
// dropout (the forward's Philox stream or a caller's dropout_mask), fp32 tensors, head dims other than
// 128 / 64, strided operands.  The reference gets these by autograd through its composite
// (csrc/ops/attention_ops.cpp:71-136: scores, mask, softmax, dropout, product with V); this is the
// same chain rule written out, on CUDA cores, in fp32:
//
//   w  = softmax(q k^T * scale + mask)            wd = dropout(w)            out = wd v
//   dwd = dO v^T      dw = dwd * keep / (1 - p)   ds = w o (dw - rowsum(w o dw)) * scale
//   dq = ds k         dk = ds^T q                 dv = wd^T dO
//
// One warp per query row, three passes over the row's keys (row max and sum; rowsum(w o dw); the
// gradients).  dq is accumulated in registers; dk and dv, which many rows (and the query heads of a GQA
// group) contribute to, are accumulated with atomic adds into fp32 scratch and rounded by a second
// kernel.  A slow path by design: O(Lq * Lk * D) on CUDA cores three times over, atomics in the order
// the hardware takes them (so not bit-reproducible run to run, unlike the fused kernels).
#include <cmath>

#include "sdpa_common.cuh"

namespace pb {
namespace {

constexpr int kRowsPerBlock = 4;
constexpr int kMaxD = 256;

struct GeneralBwdParams {
    const void* q;
    const void* k;
    const void* v;
    const void* dout;
    void* dq;
    float* dk32;
    float* dv32;
    const void* mask;
    const void* dmask;
    int mask_kind, dmask_kind;
    int B, Hq, Hkv, Lq, Lk, D;
    int64_t qs[3], ks[3], vs[3], dos[3], ms[4], ds[4];
    int causal;
    float scale;
    float keep, inv_keep;
    float one_minus_p_scalar;
    int dropout;      // 0 none, 1 Philox, 2 given mask
    uint64_t seed, sequence;
};

template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
sdpa_bwd_general_kernel(const GeneralBwdParams p) {
    __shared__ float sq[kRowsPerBlock][kMaxD];
    __shared__ float sdo[kRowsPerBlock][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qi = blockIdx.x * kRowsPerBlock + warp;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int D = p.D;
    if (qi >= p.Lq) return;

    const T* qrow = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + int64_t(qi) * p.qs[2];
    const T* dorow = static_cast<const T*>(p.dout) + b * p.dos[0] + h * p.dos[1] + int64_t(qi) * p.dos[2];
    for (int d = lane; d < D; d += 32) {
        sq[warp][d] = to_f32<T>(qrow[d]);
        sdo[warp][d] = to_f32<T>(dorow[d]);
    }
    __syncwarp();
    const int k_end = p.causal ? min(p.Lk, qi + 1) : p.Lk;   // top-left aligned: keys 0..qi
    const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
    const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
    const int64_t row = (int64_t(b) * p.Hq + h) * p.Lq + qi;

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
    // what dropout multiplies weight `key` of this row by (1 without dropout), as the forward did
    auto keep_factor = [&](int key) -> float {
        if (p.dropout == 1) {
            const uint64_t idx = uint64_t(row) * uint64_t(p.Lk) + uint64_t(key);
            const float u = float(philox2x32_r0(p.seed, p.sequence, idx) >> 8) * (1.0f / 16777216.0f);
            return u < p.keep ? p.inv_keep : 0.f;
        }
        if (p.dropout == 2) {
            const int64_t mo = b * p.ds[0] + h * p.ds[1] + int64_t(qi) * p.ds[2] + int64_t(key) * p.ds[3];
            float mv;
            if (p.dmask_kind == 1) mv = static_cast<const unsigned char*>(p.dmask)[mo] ? 1.f : 0.f;
            else if (p.dmask_kind == 2) mv = to_f32<T>(static_cast<const T*>(p.dmask)[mo]);
            else mv = static_cast<const float*>(p.dmask)[mo];
            return mv / p.one_minus_p_scalar;
        }
        return 1.f;
    };
    auto dot_do_v = [&](int key) -> float {
        const T* vrow = vbase + int64_t(key) * p.vs[2];
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(sdo[warp][d], to_f32<T>(vrow[d]), dot);
        return dot;
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
    float acc[kMaxD / 32];
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) acc[i] = 0.f;
    T* dqrow = static_cast<T*>(p.dq) + row * D;
    if (!(l > 0.f)) {   // every key masked out: the forward row is NaN, and so is its gradient (0 * inf) in the reference
        for (int d = lane; d < D; d += 32) dqrow[d] = from_f32<T>(__int_as_float(0x7fc00000));
        return;
    }
    const float inv = 1.0f / l;
    auto weight = [&](float s) -> float { return s == -INFINITY ? 0.f : expf(s - m) * inv; };

    // pass 2: delta = sum_j w_j * dw_j
    float delta = 0.f;
    for (int k0 = 0; k0 < k_end; k0 += 32) {
        const int key = k0 + lane;
        if (key < k_end) {
            const float w = weight(score(key));
            if (w != 0.f) delta = fmaf(w, dot_do_v(key) * keep_factor(key), delta);
        }
    }
    delta = warp_sum(delta);

    // pass 3: dq in registers, dk and dv into the fp32 accumulators
    float* dkb = p.dk32 + ((int64_t(b) * p.Hkv + hk) * p.Lk) * D;
    float* dvb = p.dv32 + ((int64_t(b) * p.Hkv + hk) * p.Lk) * D;
    for (int k0 = 0; k0 < k_end; k0 += 32) {
        const int key = k0 + lane;
        float ds = 0.f, wd = 0.f;
        if (key < k_end) {
            const float w = weight(score(key));
            if (w != 0.f) {
                const float kf = keep_factor(key);
                ds = w * (dot_do_v(key) * kf - delta) * p.scale;
                // the weight the forward multiplied V by: rounded to the dtype, then dropout (sdpa_weights.cu)
                wd = round_to<T>(w);
                if (p.dropout == 1) wd = kf != 0.f ? round_to<T>(wd * p.inv_keep) : 0.f;
                else if (p.dropout == 2) wd = round_to<T>(round_to<T>(wd * (kf * p.one_minus_p_scalar)) / p.one_minus_p_scalar);
            }
        }
        const int valid = min(32, k_end - k0);
        for (int j = 0; j < valid; ++j) {
            const float dsj = __shfl_sync(0xffffffffu, ds, j);
            const float wdj = __shfl_sync(0xffffffffu, wd, j);
            if (dsj == 0.f && wdj == 0.f) continue;   // uniform across the warp
            const T* krow = kbase + int64_t(k0 + j) * p.ks[2];
            float* dkrow = dkb + int64_t(k0 + j) * D;
            float* dvrow = dvb + int64_t(k0 + j) * D;
#pragma unroll
            for (int i = 0; i < kMaxD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    acc[i] = fmaf(dsj, to_f32<T>(krow[d]), acc[i]);
                    if (dsj != 0.f) atomicAdd(dkrow + d, dsj * sq[warp][d]);
                    if (wdj != 0.f) atomicAdd(dvrow + d, wdj * sdo[warp][d]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dqrow[d] = from_f32<T>(acc[i]);
    }
}

template <typename T>
__global__ void round_pair_kernel(const float* __restrict__ a32, const float* __restrict__ b32, T* __restrict__ a,
                                  T* __restrict__ b, int64_t n) {
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        a[i] = from_f32<T>(a32[i]);
        b[i] = from_f32<T>(b32[i]);
    }
}

}  // namespace
}  // namespace pb

using pb::fail;

extern "C" int paras_b200_sdpa_bwd_general(const paras_sdpa_args* a, const void* dout, const int64_t* dout_strides,
                                           void* dq, void* dk, void* dv) {
    pb::NvtxRange range("paras_b200_sdpa_bwd_general");
    if (!a || !dout || !dout_strides || !dq || !dk || !dv || !a->q || !a->k || !a->v)
        return fail(PARAS_E_INVALID, "paras sdpa backward: null pointer");
    if (a->dtype != PARAS_F32 && a->dtype != PARAS_BF16 && a->dtype != PARAS_F16)
        return fail(PARAS_E_INVALID, "paras sdpa backward: bad dtype %d", a->dtype);
    if (a->B < 0 || a->Hq < 1 || a->Hkv < 1 || a->Hq % a->Hkv || a->Lq < 0 || a->Lk < 0 || a->D < 1)
        return fail(PARAS_E_INVALID, "paras sdpa backward: bad shape");
    if (a->D > pb::kMaxD)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: head dim %d exceeds kernel limit %d", a->D, pb::kMaxD);
    if (a->B > 65535 || a->Hq > 65535)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: batch or heads exceed the grid limit");
    if (!(a->dropout_p >= 0.0) || a->dropout_p >= 1.0)
        return fail(PARAS_E_INVALID, "paras sdpa backward: dropout_p must be in [0, 1), got %g", a->dropout_p);
    if (a->mask && (a->mask_kind < 1 || a->mask_kind > 3))
        return fail(PARAS_E_INVALID, "paras sdpa backward: bad mask kind %d", a->mask_kind);
    if (a->dropout_mask && (a->dropout_mask_kind < 1 || a->dropout_mask_kind > 3))
        return fail(PARAS_E_INVALID, "paras sdpa backward: bad dropout mask kind %d", a->dropout_mask_kind);
    int st;
    pb::Gpu* g = pb::use_gpu(a->gpu, &st);
    if (!g) return st;
    cudaStream_t s = pb::pick_stream(g, a->stream);
    const size_t es = a->dtype == PARAS_F32 ? 4 : 2;
    const int64_t nq = int64_t(a->B) * a->Hq * a->Lq * a->D, nkv = int64_t(a->B) * a->Hkv * a->Lk * a->D;
    if (nq == 0 && nkv == 0) return PARAS_OK;
    if (a->Lq == 0 || a->B == 0) {   // no query contributes: dk = dv = 0
        PB_CUDA(cudaMemsetAsync(dk, 0, size_t(nkv) * es, s));
        PB_CUDA(cudaMemsetAsync(dv, 0, size_t(nkv) * es, s));
        return PARAS_OK;
    }
    if (a->Lk == 0) {                // no key: the forward output is 0 and so is dq
        PB_CUDA(cudaMemsetAsync(dq, 0, size_t(nq) * es, s));
        return PARAS_OK;
    }
    void* scratch = nullptr;
    st = paras_b200_malloc_async(a->gpu, 2 * size_t(nkv) * sizeof(float), s, &scratch);
    if (st != PARAS_OK) return st;
    PB_CUDA(cudaMemsetAsync(scratch, 0, 2 * size_t(nkv) * sizeof(float), s));

    pb::GeneralBwdParams p{};
    p.q = a->q; p.k = a->k; p.v = a->v; p.dout = dout; p.dq = dq;
    p.dk32 = static_cast<float*>(scratch);
    p.dv32 = p.dk32 + nkv;
    p.mask = a->mask; p.mask_kind = a->mask ? a->mask_kind : 0;
    p.dmask = a->dropout_mask; p.dmask_kind = a->dropout_mask_kind;
    p.B = a->B; p.Hq = a->Hq; p.Hkv = a->Hkv; p.Lq = a->Lq; p.Lk = a->Lk; p.D = a->D;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = a->q_strides[i]; p.ks[i] = a->k_strides[i]; p.vs[i] = a->v_strides[i]; p.dos[i] = dout_strides[i];
    }
    for (int i = 0; i < 4; ++i) { p.ms[i] = a->mask_strides[i]; p.ds[i] = a->dropout_mask_strides[i]; }
    p.causal = a->causal;
    p.scale = pb::effective_scale(*a);
    p.keep = float(1.0 - a->dropout_p);
    p.inv_keep = 1.0f / p.keep;
    float omp = float(1.0 - a->dropout_p);   // the divisor the forward wrapped into a 0-dim tensor of the dtype
    if (a->dtype == PARAS_BF16) omp = __bfloat162float(__float2bfloat16_rn(omp));
    else if (a->dtype == PARAS_F16) omp = __half2float(__float2half_rn(omp));
    p.one_minus_p_scalar = omp;
    p.dropout = a->dropout_p > 0.0 ? (a->dropout_mask ? 2 : 1) : 0;
    p.seed = a->rng_seed; p.sequence = a->rng_sequence;

    dim3 grid((a->Lq + pb::kRowsPerBlock - 1) / pb::kRowsPerBlock, a->Hq, a->B);
    const int threads = pb::kRowsPerBlock * 32;
    const int cblocks = int(std::min<int64_t>((nkv + 255) / 256, 148 * 8));
    switch (a->dtype) {
        case PARAS_F32:
            pb::sdpa_bwd_general_kernel<float><<<grid, threads, 0, s>>>(p);
            pb::round_pair_kernel<float><<<cblocks, 256, 0, s>>>(p.dk32, p.dv32, static_cast<float*>(dk), static_cast<float*>(dv), nkv);
            break;
        case PARAS_BF16:
            pb::sdpa_bwd_general_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(p);
            pb::round_pair_kernel<__nv_bfloat16><<<cblocks, 256, 0, s>>>(p.dk32, p.dv32, static_cast<__nv_bfloat16*>(dk),
                                                                          static_cast<__nv_bfloat16*>(dv), nkv);
            break;
        default:
            pb::sdpa_bwd_general_kernel<__half><<<grid, threads, 0, s>>>(p);
            pb::round_pair_kernel<__half><<<cblocks, 256, 0, s>>>(p.dk32, p.dv32, static_cast<__half*>(dk), static_cast<__half*>(dv), nkv);
            break;
    }
    st = cudaGetLastError() == cudaSuccess ? PARAS_OK : fail(PARAS_E_CUDA, "paras sdpa backward: kernel launch failed");
    const int st2 = paras_b200_free_async(a->gpu, scratch, s);
    return st != PARAS_OK ? st : st2;
}
