// Attention backward (the gradient the reference obtains by autograd through its composite
// sdpa_math, csrc/ops/attention_ops.cpp:71-136: mm / mul / masked_fill / softmax / mm, each with
// 16-bit intermediates).  Not a fused kernel: the row statistics the forward pass returns (lse)
// make the probabilities a pure element-wise function of the scores, so the gradient is five
// batched GEMMs on the tcgen05 GEMM of gemm_tc.cu, per kv-head group, with the element-wise
// steps in the epilogues of two of them:
//
//   P  = exp(Q K^T * scale - lse[row])        [R, Lk]   R = (Hq/Hkv) * Lq rows: the group's query heads
//                                                       stacked; causal entries zeroed (GEMM epilogue)
//   dV = P^T dO                               [Lk, D]   (sums over the group's heads by construction)
//   dS = P o (dO V^T - delta[row]) * scale    [R, Lk]   delta = rowsum(dO o O) (GEMM epilogue)
//   dK = dS^T Q                               [Lk, D]
//   dQ = dS K                                 [R, D]
//
// P and dS are materialised for a chunk of groups at a time (about 1 GB each), so the work is
// bound by HBM traffic on those two matrices, not by the tensor pipe.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "gemm_internal.cuh"
#include "sdpa_common.cuh"

namespace pb {
namespace {

// delta[row] = sum_d dO[row, d] * O[row, d].  LPR lanes share a row (16 bytes per lane and pass), so
// a warp takes 32 / LPR rows at a time and no lane idles on short head dims.
template <typename T, int LPR>
__global__ void sdpa_bwd_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out,
                                      float* __restrict__ delta, int64_t rows, int D) {
    constexpr int N = Vec16<T>::N;
    constexpr int kRowsPerWarp = 32 / LPR;
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR, l = lane % LPR;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row0 = warp * kRowsPerWarp; row0 < rows; row0 += nwarps * kRowsPerWarp) {
        const int64_t row = row0 + sub;
        float acc = 0.f;
        if (row < rows) {
            const T* a = dout + row * D;
            const T* b = out + row * D;
            for (int d = l * N; d < D; d += LPR * N) {
                const Vec16<T> x = ld16(a + d), y = ld16(b + d);
#pragma unroll
                for (int e = 0; e < N; ++e) acc = fmaf(to_f32<T>(x.v[e]), to_f32<T>(y.v[e]), acc);
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l == 0 && row < rows) delta[row] = acc;
    }
}

template <typename T>
void launch_delta(const void* dout, const void* out, float* delta, int64_t rows, int D, int sms, cudaStream_t s) {
    const T* a = static_cast<const T*>(dout);
    const T* b = static_cast<const T*>(out);
    if (D <= 64) sdpa_bwd_delta_kernel<T, 8><<<sms * 8, 256, 0, s>>>(a, b, delta, rows, D);
    else if (D <= 128) sdpa_bwd_delta_kernel<T, 16><<<sms * 8, 256, 0, s>>>(a, b, delta, rows, D);
    else sdpa_bwd_delta_kernel<T, 32><<<sms * 8, 256, 0, s>>>(a, b, delta, rows, D);
}

}  // namespace
}  // namespace pb

using pb::fail;
using pb::Gpu;

extern "C" int paras_b200_sdpa_bwd(const paras_sdpa_bwd_args* a) {
    pb::NvtxRange range("paras_b200_sdpa_bwd");
    using namespace pb;
    if (!a) return fail(PARAS_E_INVALID, "paras sdpa backward: null argument block");
    if (a->dtype != PARAS_BF16 && a->dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: bfloat16 or float16 tensors");
    if (a->B < 0 || a->Hq < 0 || a->Hkv < 0 || a->Lq < 0 || a->Lk < 0 || a->D < 0)
        return fail(PARAS_E_INVALID, "paras sdpa backward: negative dimension");
    if (a->Hkv == 0 ? a->Hq != 0 : (a->Hq % a->Hkv) != 0)
        return fail(PARAS_E_INVALID, "paras sdpa backward: query heads must be a multiple of key/value heads");
    int st;
    Gpu* g = use_gpu(a->gpu, &st);
    if (!g) return st;
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0 || int64_t(a->B) * a->Hkv * a->Lk * a->D == 0) {
        // nothing flows: gradients of empty tensors are empty, of unreached keys zero
        cudaStream_t s0 = pick_stream(g, a->stream);
        const size_t es0 = 2;
        if (a->dq && int64_t(a->B) * a->Hq * a->Lq * a->D)
            PB_CUDA(cudaMemsetAsync(a->dq, 0, size_t(a->B) * a->Hq * a->Lq * a->D * es0, s0));
        if (a->dk && int64_t(a->B) * a->Hkv * a->Lk * a->D) {
            PB_CUDA(cudaMemsetAsync(a->dk, 0, size_t(a->B) * a->Hkv * a->Lk * a->D * es0, s0));
            PB_CUDA(cudaMemsetAsync(a->dv, 0, size_t(a->B) * a->Hkv * a->Lk * a->D * es0, s0));
        }
        return PARAS_OK;
    }
    if (!a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv)
        return fail(PARAS_E_INVALID, "paras sdpa backward: null pointer");
    const int r = a->Hq / a->Hkv;
    const int64_t R = int64_t(r) * a->Lq;
    if (a->D % 8 || R > INT32_MAX)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: head dim must be a multiple of 8 (16-byte rows)");
    for (const void* ptr : {a->q, a->k, a->v, a->out, a->dout, (const void*)a->dq, (const void*)a->dk, (const void*)a->dv})
        if (reinterpret_cast<uintptr_t>(ptr) & 15u)
            return fail(PARAS_E_UNSUPPORTED, "paras sdpa backward: tensors must be 16-byte aligned");
    cudaStream_t s = pick_stream(g, a->stream);
    const size_t es = 2;
    const int64_t groups = int64_t(a->B) * a->Hkv;     // (batch, kv head): its r query heads are adjacent
    const int64_t rows = groups * R;

    // Head dim 128 / 64: the fused kernels; their only scratch is two statistics per query row.
    if (!(a->reserved & PARAS_SDPA_BWD_COMPOSITE) && sdpa_bwd_tc_supported(g, *a)) {
        void* dmem = nullptr;
        st = paras_b200_malloc_async(a->gpu, sdpa_bwd_tc_scratch_bytes(*a), s, &dmem);
        if (st != PARAS_OK) return st;
        st = sdpa_bwd_tc_launch(g, *a, static_cast<float*>(dmem), s);   // the dQ kernel fills the row statistics
        const int st2 = paras_b200_free_async(a->gpu, dmem, s);
        return st != PARAS_OK ? st : st2;
    }
    if (a->Lk % 8)
        return fail(PARAS_E_UNSUPPORTED,
                    "paras sdpa backward: this head dim takes the composite path, which needs a key length "
                    "that is a multiple of 8 (16-byte rows)");

    // scratch: delta [rows] fp32, S/P and dP/dS for a chunk of groups
    const size_t mat_bytes_per_group = size_t(R) * a->Lk * es;
    int64_t chunk = std::max<int64_t>(1, (int64_t(1) << 30) / int64_t(std::max<size_t>(mat_bytes_per_group, 1)));
    chunk = std::min(chunk, groups);
    const size_t delta_bytes = (size_t(rows) * sizeof(float) + 255) & ~size_t(255);
    const size_t mat_bytes = (mat_bytes_per_group * size_t(chunk) + 255) & ~size_t(255);
    void* scratch = nullptr;
    st = paras_b200_malloc_async(a->gpu, delta_bytes + 2 * mat_bytes, s, &scratch);
    if (st != PARAS_OK) return st;
    float* delta = static_cast<float*>(scratch);
    char* smat = static_cast<char*>(scratch) + delta_bytes;
    char* dpmat = smat + mat_bytes;

    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const float scale = float(a->scale);
    auto run = [&]() -> int {
        if (a->dtype == PARAS_BF16) launch_delta<__nv_bfloat16>(a->dout, a->out, delta, rows, a->D, sms, s);
        else launch_delta<__half>(a->dout, a->out, delta, rows, a->D, sms, s);
        PB_LAUNCH_CHECK("sdpa_bwd_delta_kernel");
        for (int64_t g0 = 0; g0 < groups; g0 += chunk) {
            const int64_t n = std::min(chunk, groups - g0);
            const char* q = static_cast<const char*>(a->q) + size_t(g0) * R * a->D * es;
            const char* dO = static_cast<const char*>(a->dout) + size_t(g0) * R * a->D * es;
            const char* k = static_cast<const char*>(a->k) + size_t(g0) * a->Lk * a->D * es;
            const char* v = static_cast<const char*>(a->v) + size_t(g0) * a->Lk * a->D * es;
            char* dq = static_cast<char*>(a->dq) + size_t(g0) * R * a->D * es;
            char* dk = static_cast<char*>(a->dk) + size_t(g0) * a->Lk * a->D * es;
            char* dv = static_cast<char*>(a->dv) + size_t(g0) * a->Lk * a->D * es;
            auto gemm = [&](const void* A, int a_layout, int64_t lda, int64_t sa, const void* Bm, int b_layout,
                            int64_t ldb, int64_t sb, void* C, int64_t ldc, int64_t sc, int64_t M, int64_t N,
                            int64_t K, const GemmExtra* ex = nullptr) -> int {
                paras_gemm_args ga{};
                ga.a = A; ga.b = Bm; ga.c = C;
                ga.M = M; ga.N = N; ga.K = K;
                ga.lda = lda; ga.ldb = ldb; ga.ldc = ldc;
                ga.batch = n; ga.stride_a = sa; ga.stride_b = sb; ga.stride_c = sc;
                ga.dtype = a->dtype; ga.a_layout = a_layout; ga.b_layout = b_layout;
                ga.epilogue = PARAS_GEMM_EPI_NONE; ga.gpu = a->gpu; ga.stream = s;
                return gemm_run(&ga, ex);
            };
            const int64_t qs = R * a->D, ks = int64_t(a->Lk) * a->D, ms = R * a->Lk;
            int rc;
            // P = exp(Q K^T * scale - lse)
            GemmExtra ex{};
            ex.epilogue = 3; ex.row_stat = a->lse + g0 * R; ex.Lq = a->Lq; ex.causal = a->causal; ex.scale = scale;
            // tiles of P and dS no query sees are left unwritten: the three reductions below skip them.
            // With more keys than queries a key tile past the last query still needs its zeros.
            ex.tile_skip = a->Lk <= a->Lq;
            if ((rc = gemm(q, PARAS_GEMM_A_MK, a->D, qs, k, PARAS_GEMM_B_NK, a->D, ks, smat, a->Lk, ms, R, a->Lk, a->D, &ex)) != PARAS_OK) return rc;
            // dV = P^T dO  (under a causal mask the query rows before a key tile hold only zeros: skipped)
            GemmExtra skip{};
            skip.epilogue = 0; skip.Lq = a->Lq; skip.causal = a->causal; skip.k_skip = 2;
            if ((rc = gemm(smat, PARAS_GEMM_A_KM, a->Lk, ms, dO, PARAS_GEMM_B_KN, a->D, qs, dv, a->D, ks, a->Lk, a->D, R, &skip)) != PARAS_OK) return rc;
            // dS = P o (dO V^T - delta) * scale
            ex.epilogue = 4; ex.row_stat = delta + g0 * R; ex.prob = smat; ex.prob_ld = a->Lk;
            if ((rc = gemm(dO, PARAS_GEMM_A_MK, a->D, qs, v, PARAS_GEMM_B_NK, a->D, ks, dpmat, a->Lk, ms, R, a->Lk, a->D, &ex)) != PARAS_OK) return rc;
            // dK = dS^T Q
            if ((rc = gemm(dpmat, PARAS_GEMM_A_KM, a->Lk, ms, q, PARAS_GEMM_B_KN, a->D, qs, dk, a->D, ks, a->Lk, a->D, R, &skip)) != PARAS_OK) return rc;
            // dQ = dS K
            skip.k_skip = 1;  // keys past a query tile's last row
            if ((rc = gemm(dpmat, PARAS_GEMM_A_MK, a->Lk, ms, k, PARAS_GEMM_B_KN, a->D, ks, dq, a->D, qs, R, a->D, a->Lk, &skip)) != PARAS_OK) return rc;
        }
        return PARAS_OK;
    };
    st = run();
    const int st2 = paras_b200_free_async(a->gpu, scratch, s);
    return st != PARAS_OK ? st : st2;
}
