// Shared helpers of libparas_b200: status codes, thread-local error text, device/stream
// resolution and small device-side conversion utilities.  No torch, no C++ exceptions
// across the ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "paras_b200.h"

namespace pb {

// Records a message for paras_b200_last_error() of this thread and returns `code`.
int fail(int code, const char* fmt, ...);
void set_last_kernel(const char* name);

// Per-GPU state owned by runtime.cu.
struct Gpu {
    int ordinal = -1;
    cudaStream_t stream = nullptr;     // the library's non-blocking stream
    cudaStream_t copy_stream = nullptr;
    cudaMemPool_t pool = nullptr;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
    char name[256] = {0};
    // Status word in mapped pinned host memory: kernels whose bounded waits run out
    // write a non-zero code here instead of trapping or spinning.
    int* status_host = nullptr;
    int* status_dev = nullptr;
    // Host-side cap on the bytes the pool may have handed out (0 = none): an allocation that would
    // go past it fails with PARAS_E_NOMEM before any CUDA call.  For sharing a GPU with another
    // owner, and for exercising the out-of-memory path without exhausting a GPU.
    size_t limit_bytes = 0;
};

// Profiler range around a public entry point, active when PARAS_NVTX is set (the reference has only
// its PTSYCL_LOG op trace, core/log.h:30-60).  Without a profiler attached NVTX calls do nothing.
struct NvtxRange {
    explicit NvtxRange(const char* name);
    ~NvtxRange();
    bool on;
};

// Returns PARAS_E_TIMEOUT (and clears the word) when a kernel on `g` reported that one of
// its bounded waits gave up; PARAS_OK otherwise.
int check_status_word(Gpu* g);
// True when `p` lies in page-locked host memory (allocated by this library or registered with CUDA).
bool host_ptr_is_pinned(const void* p);

// Makes `gpu` current on the calling thread and returns its state; nullptr (and an error
// message) when the ordinal is bad or there is no device.
Gpu* use_gpu(int gpu, int* status);

inline cudaStream_t pick_stream(Gpu* g, void* stream) {
    return stream ? static_cast<cudaStream_t>(stream) : g->stream;
}

#define PB_CUDA(call)                                                                    \
    do {                                                                                 \
        cudaError_t e_ = (call);                                                         \
        if (e_ != cudaSuccess)                                                           \
            return ::pb::fail(PARAS_E_CUDA, "paras_b200: %s: %s", #call,                  \
                              cudaGetErrorString(e_));                                   \
    } while (0)

#define PB_LAUNCH_CHECK(what)                                                            \
    do {                                                                                 \
        cudaError_t e_ = cudaGetLastError();                                             \
        if (e_ != cudaSuccess)                                                           \
            return ::pb::fail(PARAS_E_CUDA, "paras_b200: launch of %s failed: %s", what, \
                              cudaGetErrorString(e_));                                   \
    } while (0)

inline size_t dtype_size(int dt) { return dt == PARAS_F32 ? 4 : 2; }

// ---- device-side scalar conversions -------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) {
    return __float2half_rn(v);
}

// Rounds an fp32 value to T and back: the reference's "result cast to the tensor dtype".
template <typename T> __device__ __forceinline__ float round_to(float v) {
    return to_f32<T>(from_f32<T>(v));
}

// 16-byte vector of T.
template <typename T> struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
    return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
template <typename T>
__device__ __forceinline__ void st16_stream(T* p, const Vec16<T>& r) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
}

// Rotary embedding on packed 16-bit pairs: the two products and the sum each round once to the
// tensors' dtype, which is what the reference's three binary kernels do (pointwise_ops.cpp:62-85).
template <bool BF16> struct Pair16;
template <> struct Pair16<true> {
    using T2 = __nv_bfloat162;
};
template <> struct Pair16<false> {
    using T2 = __half2;
};
// x1, x2: eight elements d.. and d+64.. of a row; c1, s1 / c2, s2: cos and sin at the same columns.
// out1 = x1*c1 + (-x2)*s1, out2 = x2*c2 + x1*s2  (x*cos + rotate_half(x)*sin, fused_ops.cpp:234-267)
template <bool BF16>
__device__ __forceinline__ void rope_rotate8(uint4& x1, uint4& x2, const uint4& c1, const uint4& s1,
                                             const uint4& c2, const uint4& s2) {
    using T2 = typename Pair16<BF16>::T2;
    T2* a = reinterpret_cast<T2*>(&x1);
    T2* b = reinterpret_cast<T2*>(&x2);
    const T2* pc1 = reinterpret_cast<const T2*>(&c1);
    const T2* ps1 = reinterpret_cast<const T2*>(&s1);
    const T2* pc2 = reinterpret_cast<const T2*>(&c2);
    const T2* ps2 = reinterpret_cast<const T2*>(&s2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // (_rn forms: no contraction of a product and the sum into a fused multiply-add, which would
        // skip the product's rounding)
        const T2 o1 = __hadd2_rn(__hmul2_rn(a[i], pc1[i]), __hmul2_rn(__hneg2(b[i]), ps1[i]));
        const T2 o2 = __hadd2_rn(__hmul2_rn(b[i], pc2[i]), __hmul2_rn(a[i], ps2[i]));
        a[i] = o1;
        b[i] = o2;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace pb
