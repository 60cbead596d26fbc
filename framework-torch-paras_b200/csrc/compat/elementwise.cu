// Memory-bound elementwise kernels: SwiGLU forward/backward, rotate_half, strided
// copy-with-cast and fill.
//
// SwiGLU replaces the reference's paras::swiglu lambda (csrc/ops/fused_ops.cpp:162-194,
// one generic grid-stride thread per element with per-element div/mod index math, double
// arithmetic) and the torch_paras::swiglu composite (csrc/ops/rms_swiglu_ops.cpp:83-86:
// silu.out then mul.out, two passes over HBM) with ONE pass: 128-bit streaming loads of
// gate and up, fp32 math, 128-bit streaming store.  Algorithmic traffic 3*n*sizeof(T).
#include <algorithm>

#include "common.cuh"

namespace pb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <typename T> __device__ __forceinline__ float silu_f32(float g) {
    if constexpr (sizeof(T) == 4) {
        return g / (1.0f + expf(-g));
    } else {
        return __fdividef(g, 1.0f + __expf(-g));
    }
}

template <typename T, int MODE>
__device__ __forceinline__ T swiglu_one(T g, T u) {
    const float gf = to_f32<T>(g);
    const float uf = to_f32<T>(u);
    float s = silu_f32<T>(gf);
    if constexpr (MODE == PARAS_ROUND_PER_OP) s = round_to<T>(s);
    return from_f32<T>(s * uf);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_vec_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                      int64_t nvec) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = int64_t(gridDim.x) * kThreads * kUnroll;
    for (int64_t base = int64_t(blockIdx.x) * kThreads * kUnroll + threadIdx.x; base < nvec;
         base += stride) {
        Vec16<T> g[kUnroll], u[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const int64_t i = base + int64_t(k) * kThreads;
            if (i < nvec) {
                g[k] = ld16_stream(gate + i * N);
                u[k] = ld16_stream(up + i * N);
            }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const int64_t i = base + int64_t(k) * kThreads;
            if (i < nvec) {
                Vec16<T> o;
#pragma unroll
                for (int e = 0; e < N; ++e) o.v[e] = swiglu_one<T, MODE>(g[k].v[e], u[k].v[e]);
                st16_stream(out + i * N, o);
            }
        }
    }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                         T* __restrict__ out, int64_t begin, int64_t n) {
    for (int64_t i = begin + int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * kThreads)
        out[i] = swiglu_one<T, MODE>(gate[i], up[i]);
}

// dgate = dy*u*s*(1+g*(1-s)), dup = dy*g*s with s = sigmoid(g)  (fused_ops.cpp:196-229)
template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                  T* __restrict__ dgate, T* __restrict__ dup, int64_t first, int64_t n) {
    for (int64_t i = first + int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * kThreads) {
        const float d = to_f32<T>(dy[i]), g = to_f32<T>(gate[i]), u = to_f32<T>(up[i]);
        const float s = 1.0f / (1.0f + expf(-g));
        dup[i] = from_f32<T>(d * g * s);
        dgate[i] = from_f32<T>(d * u * (s * (1.0f + g * (1.0f - s))));
    }
}

// The same on 16-byte vectors with streaming loads and stores, two vectors of each input in flight per
// thread (three inputs, two outputs: 5 * n * sizeof(T) bytes of HBM traffic, read once, written once).
template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                      T* __restrict__ dgate, T* __restrict__ dup, int64_t nvec) {
    constexpr int N = Vec16<T>::N;
    constexpr int U = 2;
    const int64_t stride = int64_t(gridDim.x) * kThreads * U;
    for (int64_t base = int64_t(blockIdx.x) * kThreads * U + threadIdx.x; base < nvec; base += stride) {
        Vec16<T> d[U], g[U], u[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int64_t i = base + int64_t(k) * kThreads;
            if (i < nvec) {
                d[k] = ld16_stream(dy + i * N);
                g[k] = ld16_stream(gate + i * N);
                u[k] = ld16_stream(up + i * N);
            }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int64_t i = base + int64_t(k) * kThreads;
            if (i < nvec) {
                Vec16<T> og, ou;
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float de = to_f32<T>(d[k].v[e]), ge = to_f32<T>(g[k].v[e]), ue = to_f32<T>(u[k].v[e]);
                    // 16-bit results: the fast exponential and reciprocal are ~2 ulp of fp32, far inside the
                    // rounding to 8 or 11 bits, and halve the instruction count of a kernel that is issue-bound
                    const float sg = sizeof(T) == 4 ? 1.0f / (1.0f + expf(-ge)) : __fdividef(1.0f, 1.0f + __expf(-ge));
                    ou.v[e] = from_f32<T>(de * ge * sg);
                    og.v[e] = from_f32<T>(de * ue * (sg * (1.0f + ge * (1.0f - sg))));
                }
                st16_stream(dgate + i * N, og);
                st16_stream(dup + i * N, ou);
            }
        }
    }
}

// out[n, k] = weight[n, k] * scale[k], one rounding: the RMSNorm weight folded into the rows of the
// projection weight that follows the norm.
template <typename T>
__global__ void __launch_bounds__(kThreads)
scale_columns_kernel(const T* __restrict__ w, const T* __restrict__ scale, T* __restrict__ out, int64_t n, int64_t K) {
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        out[i] = from_f32<T>(to_f32<T>(w[i]) * to_f32<T>(scale[i % K]));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
rotate_half_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, int64_t D,
                   int backward) {
    const int64_t half = D / 2;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * kThreads) {
        const int64_t col = i % D;
        const bool lo = col < half;
        const T v = x[lo ? i + half : i - half];
        const bool neg = backward ? !lo : lo;
        out[i] = neg ? from_f32<T>(-to_f32<T>(v)) : v;
    }
}

// The same on 16-byte vectors (half a row is a whole number of vectors): vector j of the output's first
// half is minus vector j of the input's second half, and the other way round without the sign.
template <typename T>
__global__ void __launch_bounds__(kThreads)
rotate_half_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t nvec, int vec_per_half, int backward) {
    constexpr int N = Vec16<T>::N;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += int64_t(gridDim.x) * kThreads) {
        const int64_t hrow = i / vec_per_half;            // (row, half) pair
        const bool lo = (hrow & 1) == 0;                  // this vector lies in the output's first half
        Vec16<T> v = ld16_stream(x + (lo ? i + vec_per_half : i - vec_per_half) * N);
        if (backward ? !lo : lo) {
#pragma unroll
            for (int e = 0; e < N; ++e) v.v[e] = from_f32<T>(-to_f32<T>(v.v[e]));
        }
        st16_stream(out + i * N, v);
    }
}

// Rotary embedding out = x * cos + rotate_half(x) * sin for x [B, H, L, D] (element strides for
// B, H, L; unit stride on D) and cos / sin [Lmax, D] read at rows pos0 + l.  The reference composes
// this from three binary kernels that each round to the tensor dtype (pointwise_ops.cpp:62-85) around
// its exact rotate_half (fused_ops.cpp:234-267); the two products and the sum round here the same way.
// One thread per pair (d, d + D/2).  `out` is dense [B, H, L, D].
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* __restrict__ x, const T* __restrict__ cosv, const T* __restrict__ sinv, T* __restrict__ out,
            int64_t n_pairs, int H, int L, int D, int64_t sb, int64_t sh, int64_t sl, int64_t pos0) {
    const int half = D / 2;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n_pairs; i += int64_t(gridDim.x) * kThreads) {
        const int d = int(i % half);
        int64_t r = i / half;
        const int l = int(r % L);
        r /= L;
        const int h = int(r % H);
        const int64_t b = r / H;
        const T* xr = x + b * sb + h * sh + int64_t(l) * sl;
        const T* cr = cosv + (pos0 + l) * D;
        const T* sr = sinv + (pos0 + l) * D;
        const float x1 = to_f32<T>(xr[d]), x2 = to_f32<T>(xr[d + half]);
        T* o = out + ((b * H + h) * int64_t(L) + l) * D;
        // (__fmul_rn / __fadd_rn: no contraction into a fused multiply-add, which would skip a rounding)
        o[d] = from_f32<T>(__fadd_rn(round_to<T>(__fmul_rn(x1, to_f32<T>(cr[d]))),
                                     round_to<T>(__fmul_rn(-x2, to_f32<T>(sr[d])))));
        o[d + half] = from_f32<T>(__fadd_rn(round_to<T>(__fmul_rn(x2, to_f32<T>(cr[d + half]))),
                                            round_to<T>(__fmul_rn(x1, to_f32<T>(sr[d + half])))));
    }
}

// The same for 16-bit tensors whose rows can be read 16 bytes at a time: a thread takes eight
// columns d.. and the matching eight at d + D/2 (six 128-bit loads, two stores, packed arithmetic).
template <bool BF16>
__global__ void __launch_bounds__(kThreads)
rope_vec16_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ cosv, const uint16_t* __restrict__ sinv,
                  uint16_t* __restrict__ out, int64_t n_units, int H, int L, int D, int64_t sb, int64_t sh, int64_t sl,
                  int64_t pos0) {
    const int upr = D / 16;   // 8-element units per half row
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n_units; i += int64_t(gridDim.x) * kThreads) {
        const int u = int(i % upr);
        int64_t r = i / upr;
        const int l = int(r % L);
        r /= L;
        const int h = int(r % H);
        const int64_t b = r / H;
        const uint16_t* xr = x + b * sb + h * sh + int64_t(l) * sl;
        const uint16_t* cr = cosv + (pos0 + l) * D;
        const uint16_t* sr = sinv + (pos0 + l) * D;
        uint4 x1 = __ldcs(reinterpret_cast<const uint4*>(xr + 8 * u));
        uint4 x2 = __ldcs(reinterpret_cast<const uint4*>(xr + D / 2 + 8 * u));
        rope_rotate8<BF16>(x1, x2, __ldg(reinterpret_cast<const uint4*>(cr + 8 * u)), __ldg(reinterpret_cast<const uint4*>(sr + 8 * u)),
                           __ldg(reinterpret_cast<const uint4*>(cr + D / 2 + 8 * u)),
                           __ldg(reinterpret_cast<const uint4*>(sr + D / 2 + 8 * u)));
        uint16_t* o = out + ((b * H + h) * int64_t(L) + l) * D;
        __stcs(reinterpret_cast<uint4*>(o + 8 * u), x1);
        __stcs(reinterpret_cast<uint4*>(o + D / 2 + 8 * u), x2);
    }
}

// ---- strided copy with conversion ----------------------------------------------------
struct CopySpec {
    int ndim;
    int64_t sizes[8];
    int64_t sstr[8];
    int64_t dstr[8];
};

struct Wide {
    double d;
    long long i;
    bool is_int;
};

__device__ __forceinline__ Wide load_wide(const void* p, int code, int64_t off) {
    Wide w{0.0, 0, false};
    switch (code) {
        case PARAS_SC_F32: w.d = static_cast<const float*>(p)[off]; break;
        case PARAS_SC_BF16: w.d = __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]); break;
        case PARAS_SC_F16: w.d = __half2float(static_cast<const __half*>(p)[off]); break;
        case PARAS_SC_F64: w.d = static_cast<const double*>(p)[off]; break;
        case PARAS_SC_I64: w.i = static_cast<const long long*>(p)[off]; w.is_int = true; break;
        case PARAS_SC_I32: w.i = static_cast<const int*>(p)[off]; w.is_int = true; break;
        case PARAS_SC_I16: w.i = static_cast<const short*>(p)[off]; w.is_int = true; break;
        case PARAS_SC_I8: w.i = static_cast<const signed char*>(p)[off]; w.is_int = true; break;
        case PARAS_SC_U8: w.i = static_cast<const unsigned char*>(p)[off]; w.is_int = true; break;
        case PARAS_SC_BOOL: w.i = static_cast<const unsigned char*>(p)[off] ? 1 : 0; w.is_int = true; break;
    }
    return w;
}

__device__ __forceinline__ void store_wide(void* p, int code, int64_t off, const Wide& w) {
    const double d = w.is_int ? double(w.i) : w.d;
    const long long i = w.is_int ? w.i : (long long)(w.d);
    switch (code) {
        case PARAS_SC_F32: static_cast<float*>(p)[off] = w.is_int ? float(w.i) : float(w.d); break;
        case PARAS_SC_BF16: static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16_rn(float(d)); break;
        case PARAS_SC_F16: static_cast<__half*>(p)[off] = __float2half_rn(float(d)); break;
        case PARAS_SC_F64: static_cast<double*>(p)[off] = d; break;
        case PARAS_SC_I64: static_cast<long long*>(p)[off] = i; break;
        case PARAS_SC_I32: static_cast<int*>(p)[off] = int(i); break;
        case PARAS_SC_I16: static_cast<short*>(p)[off] = short(i); break;
        case PARAS_SC_I8: static_cast<signed char*>(p)[off] = (signed char)(i); break;
        case PARAS_SC_U8: static_cast<unsigned char*>(p)[off] = (unsigned char)(i); break;
        case PARAS_SC_BOOL:
            static_cast<unsigned char*>(p)[off] = (w.is_int ? (w.i != 0) : (w.d != 0.0)) ? 1 : 0;
            break;
    }
}

__global__ void __launch_bounds__(kThreads)
strided_copy_kernel(void* dst, int dcode, const void* src, int scode, CopySpec sp, int64_t n) {
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * kThreads) {
        int64_t rem = i, so = 0, dof = 0;
#pragma unroll 1
        for (int d = sp.ndim - 1; d >= 0; --d) {
            const int64_t q = rem / sp.sizes[d];
            const int64_t r = rem - q * sp.sizes[d];
            so += r * sp.sstr[d];
            dof += r * sp.dstr[d];
            rem = q;
        }
        store_wide(dst, dcode, dof, load_wide(src, scode, so));
    }
}

// ---- fast paths of the strided copy --------------------------------------------------------
// Rows: the innermost dimension is contiguous on both sides and a multiple of 8 elements, the element
// types are floating point (any pair of fp32 / bf16 / fp16).  A group of G lanes takes a row at a time, 8
// elements per lane and step, with 16-byte accesses; the row's offsets are worked out once per row.
template <typename T> struct Load8;
template <> struct Load8<float> {
    static __device__ __forceinline__ void run(const float* p, float (&f)[8]) {
        const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
        __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(f[4], f[5], f[6], f[7]));
    }
};
template <typename T> struct Load8 {
    static __device__ __forceinline__ void run(const T* p, float (&f)[8]) {
        const Vec16<T> v = ld16_stream(p);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = to_f32<T>(v.v[e]);
    }
    static __device__ __forceinline__ void store(T* p, const float (&f)[8]) {
        Vec16<T> v;
#pragma unroll
        for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(f[e]);
        st16_stream(p, v);
    }
};

template <typename S, typename D, int G>
__global__ void __launch_bounds__(kThreads)
row_copy8_kernel(D* __restrict__ dst, const S* __restrict__ src, CopySpec sp, int64_t rows, int64_t inner8) {
    const int64_t group = (int64_t(blockIdx.x) * kThreads + threadIdx.x) / G, ngroups = int64_t(gridDim.x) * kThreads / G;
    const int gl = threadIdx.x % G;
    for (int64_t row = group; row < rows; row += ngroups) {
        int64_t rem = row, so = 0, dof = 0;
#pragma unroll 1
        for (int d = sp.ndim - 2; d >= 0; --d) {
            const int64_t q = rem / sp.sizes[d];
            const int64_t r = rem - q * sp.sizes[d];
            so += r * sp.sstr[d];
            dof += r * sp.dstr[d];
            rem = q;
        }
        for (int64_t j = gl; j < inner8; j += G) {
            float f[8];
            Load8<S>::run(src + so + 8 * j, f);
            Load8<D>::store(dst + dof + 8 * j, f);
        }
    }
}

// Transposes: the last two dimensions change places (source unit stride on the second to last one,
// destination on the last one), same element size.  32 x 32 tiles through shared memory, so that both
// sides are read and written along their unit stride; leading dimensions are walked by blockIdx.z.
template <typename T>
__global__ void __launch_bounds__(256)
transpose_tile_kernel(T* __restrict__ dst, const T* __restrict__ src, CopySpec sp, int64_t R, int64_t C,
                      int64_t s_ld, int64_t d_ld) {
    // dst[b][r][c] = src[b][c][r] in memory terms: src element (r, c) sits at c * s_ld + r, dst at r * d_ld + c
    __shared__ T tile[32][33];
    int64_t rem = blockIdx.z, so = 0, dof = 0;
    for (int d = sp.ndim - 3; d >= 0; --d) {
        const int64_t q = rem / sp.sizes[d];
        const int64_t r = rem - q * sp.sizes[d];
        so += r * sp.sstr[d];
        dof += r * sp.dstr[d];
        rem = q;
    }
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    const int64_t r0 = int64_t(blockIdx.x) * 32, c0 = int64_t(blockIdx.y) * 32;
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int64_t c = c0 + ty + k, r = r0 + tx;            // read along r (the source's unit stride)
        if (c < C && r < R) tile[ty + k][tx] = src[so + c * s_ld + r];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int64_t r = r0 + ty + k, c = c0 + tx;            // write along c (the destination's unit stride)
        if (r < R && c < C) dst[dof + r * d_ld + c] = tile[tx][ty + k];
    }
}

__global__ void __launch_bounds__(kThreads)
fill_kernel(void* dst, int code, double value, int64_t n) {
    Wide w{value, (long long)value, false};
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * kThreads)
        store_wide(dst, code, i, w);
}

int grid_for(const Gpu* g, int64_t work_items, int per_block, int waves = 8) {
    int64_t blocks = (work_items + per_block - 1) / per_block;
    const int64_t cap = int64_t(g->sm_count > 0 ? g->sm_count : 148) * waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return int(blocks);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int MODE>
int launch_swiglu(Gpu* g, const void* gate, const void* up, void* out, int64_t n,
                  cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    const T* pg = static_cast<const T*>(gate);
    const T* pu = static_cast<const T*>(up);
    T* po = static_cast<T*>(out);
    int64_t done = 0;
    if (aligned16(gate) && aligned16(up) && aligned16(out) && n >= N) {
        const int64_t nvec = n / N;
        // One CTA-iteration moves kThreads*kUnroll vectors; the grid is a multiple of the
        // SM count so every SM streams the same share.
        const int blocks = grid_for(g, nvec, kThreads * kUnroll, 16);
        swiglu_fwd_vec_kernel<T, MODE><<<blocks, kThreads, 0, s>>>(pg, pu, po, nvec);
        PB_LAUNCH_CHECK("swiglu_fwd_vec_kernel");
        done = nvec * N;
    }
    if (done < n) {
        const int blocks = grid_for(g, n - done, kThreads);
        swiglu_fwd_scalar_kernel<T, MODE><<<blocks, kThreads, 0, s>>>(pg, pu, po, done, n);
        PB_LAUNCH_CHECK("swiglu_fwd_scalar_kernel");
    }
    return PARAS_OK;
}

int code_size(int code) {
    switch (code) {
        case PARAS_SC_F64: case PARAS_SC_I64: return 8;
        case PARAS_SC_F32: case PARAS_SC_I32: return 4;
        case PARAS_SC_BF16: case PARAS_SC_F16: case PARAS_SC_I16: return 2;
        default: return 1;
    }
}
bool is_float16_32(int code) { return code == PARAS_SC_F32 || code == PARAS_SC_BF16 || code == PARAS_SC_F16; }

template <typename S, typename D>
void launch_rows(const Gpu* g, void* dst, const void* src, const CopySpec& sp, int64_t rows, int64_t inner8, cudaStream_t s) {
    D* d = static_cast<D*>(dst);
    const S* sr = static_cast<const S*>(src);
    const int64_t work = rows * std::min<int64_t>(inner8, 32);
    const int blocks = grid_for(g, work, kThreads, 16);
    if (inner8 >= 32) row_copy8_kernel<S, D, 32><<<blocks, kThreads, 0, s>>>(d, sr, sp, rows, inner8);
    else if (inner8 >= 16) row_copy8_kernel<S, D, 16><<<blocks, kThreads, 0, s>>>(d, sr, sp, rows, inner8);
    else if (inner8 >= 8) row_copy8_kernel<S, D, 8><<<blocks, kThreads, 0, s>>>(d, sr, sp, rows, inner8);
    else if (inner8 >= 4) row_copy8_kernel<S, D, 4><<<blocks, kThreads, 0, s>>>(d, sr, sp, rows, inner8);
    else row_copy8_kernel<S, D, 2><<<blocks, kThreads, 0, s>>>(d, sr, sp, rows, inner8);
}
template <typename S>
void launch_rows_dst(const Gpu* g, void* dst, int dcode, const void* src, const CopySpec& sp, int64_t rows, int64_t inner8,
                     cudaStream_t s) {
    if (dcode == PARAS_SC_F32) launch_rows<S, float>(g, dst, src, sp, rows, inner8, s);
    else if (dcode == PARAS_SC_BF16) launch_rows<S, __nv_bfloat16>(g, dst, src, sp, rows, inner8, s);
    else launch_rows<S, __half>(g, dst, src, sp, rows, inner8, s);
}

// Picks a fast kernel for the common layouts of a copy; false = take the generic element-wise kernel.
bool copy_fast_path(const Gpu* g, void* dst, int dcode, const void* src, int scode, const CopySpec& sp_in, int64_t n,
                    cudaStream_t s) {
    if (sp_in.ndim < 1 || n < 4096) return false;
    // drop dimensions of size 1, merge neighbours that are contiguous on both sides
    CopySpec sp{};
    for (int d = 0; d < sp_in.ndim; ++d) {
        if (sp_in.sizes[d] == 1) continue;
        if (sp.ndim > 0 && sp.sstr[sp.ndim - 1] == sp_in.sstr[d] * sp_in.sizes[d] &&
            sp.dstr[sp.ndim - 1] == sp_in.dstr[d] * sp_in.sizes[d]) {
            sp.sizes[sp.ndim - 1] *= sp_in.sizes[d];
            sp.sstr[sp.ndim - 1] = sp_in.sstr[d];
            sp.dstr[sp.ndim - 1] = sp_in.dstr[d];
        } else {
            sp.sizes[sp.ndim] = sp_in.sizes[d];
            sp.sstr[sp.ndim] = sp_in.sstr[d];
            sp.dstr[sp.ndim] = sp_in.dstr[d];
            ++sp.ndim;
        }
    }
    if (sp.ndim < 1) return false;
    const int L = sp.ndim - 1;
    const int ss = code_size(scode), ds = code_size(dcode);
    auto aligned = [&](const void* base, const int64_t* str, int es) {
        if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
        for (int d = 0; d < L; ++d)
            if ((str[d] * es) % 16) return false;
        return true;
    };
    // rows of floating-point elements, unit stride on both sides
    if (is_float16_32(scode) && is_float16_32(dcode) && sp.sstr[L] == 1 && sp.dstr[L] == 1 && sp.sizes[L] % 8 == 0 &&
        aligned(src, sp.sstr, ss) && aligned(dst, sp.dstr, ds)) {
        int64_t inner = sp.sizes[L], rows = n / inner;
        if (sp.ndim == 1) {   // one long contiguous run: cut it into rows of 2048 elements (or fewer that divide it)
            int64_t chunk = 2048;
            while (chunk > 8 && inner % chunk) chunk /= 2;
            sp.ndim = 2;
            sp.sizes[0] = inner / chunk; sp.sstr[0] = chunk; sp.dstr[0] = chunk;
            sp.sizes[1] = chunk; sp.sstr[1] = 1; sp.dstr[1] = 1;
            rows = inner / chunk;
            inner = chunk;
        }
        if (scode == PARAS_SC_F32) launch_rows_dst<float>(g, dst, dcode, src, sp, rows, inner / 8, s);
        else if (scode == PARAS_SC_BF16) launch_rows_dst<__nv_bfloat16>(g, dst, dcode, src, sp, rows, inner / 8, s);
        else launch_rows_dst<__half>(g, dst, dcode, src, sp, rows, inner / 8, s);
        return true;
    }
    // the last two dimensions change places, same element size (2 or 4 bytes)
    if (sp.ndim >= 2 && scode == dcode && (ss == 2 || ss == 4) && sp.dstr[L] == 1 && sp.sstr[L - 1] == 1 &&
        sp.sstr[L] >= sp.sizes[L - 1] && sp.dstr[L - 1] >= sp.sizes[L]) {
        const int64_t R = sp.sizes[L - 1], C = sp.sizes[L];
        int64_t batch = 1;
        for (int d = 0; d < L - 1; ++d) batch *= sp.sizes[d];
        if (batch > 65535 || (C + 31) / 32 > 65535) return false;
        dim3 grid(unsigned((R + 31) / 32), unsigned((C + 31) / 32), unsigned(batch));
        if (ss == 2)
            transpose_tile_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), sp,
                                                               R, C, sp.sstr[L], sp.dstr[L - 1]);
        else
            transpose_tile_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<uint32_t*>(dst), static_cast<const uint32_t*>(src), sp,
                                                               R, C, sp.sstr[L], sp.dstr[L - 1]);
        return true;
    }
    return false;
}

}  // namespace
}  // namespace pb

using pb::fail;
using pb::Gpu;

extern "C" {

int paras_b200_swiglu_fwd(int gpu, const void* gate, const void* up, void* out, int64_t n,
                          int dtype, int mode, void* stream) {
    pb::NvtxRange range("paras_b200_swiglu_fwd");
    if (n < 0) return fail(PARAS_E_INVALID, "paras swiglu: negative element count");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras swiglu: unsupported dtype %d", dtype);
    if (mode != PARAS_ROUND_ONCE && mode != PARAS_ROUND_PER_OP)
        return fail(PARAS_E_INVALID, "paras swiglu: bad rounding mode %d", mode);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (n == 0) return PARAS_OK;
    if (!gate || !up || !out) return fail(PARAS_E_INVALID, "paras swiglu: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
#define PB_SWIGLU(T)                                                               \
    (mode == PARAS_ROUND_ONCE ? pb::launch_swiglu<T, PARAS_ROUND_ONCE>(g, gate, up, out, n, s) \
                              : pb::launch_swiglu<T, PARAS_ROUND_PER_OP>(g, gate, up, out, n, s))
    switch (dtype) {
        case PARAS_F32: return PB_SWIGLU(float);
        case PARAS_BF16: return PB_SWIGLU(__nv_bfloat16);
        default: return PB_SWIGLU(__half);
    }
#undef PB_SWIGLU
}

int paras_b200_swiglu_bwd(int gpu, const void* grad_out, const void* gate, const void* up,
                          void* grad_gate, void* grad_up, int64_t n, int dtype, void* stream) {
    pb::NvtxRange range("paras_b200_swiglu_bwd");
    if (n < 0) return fail(PARAS_E_INVALID, "paras swiglu_backward: negative element count");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras swiglu_backward: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (n == 0) return PARAS_OK;
    if (!grad_out || !gate || !up || !grad_gate || !grad_up)
        return fail(PARAS_E_INVALID, "paras swiglu_backward: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    const int64_t per = 16 / int64_t(pb::dtype_size(dtype));
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(gate) |
                          reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(grad_gate) |
                          reinterpret_cast<uintptr_t>(grad_up)) & 15u) == 0;
    const int64_t nvec = vec_ok ? n / per : 0, done = nvec * per;
    const int vblocks = nvec ? pb::grid_for(g, (nvec + 1) / 2, pb::kThreads, 16) : 0;
    const int blocks = done < n ? pb::grid_for(g, n - done, pb::kThreads) : 0;
#define PB_BWD(T)                                                                        \
    do {                                                                                 \
        if (nvec)                                                                        \
            pb::swiglu_bwd_vec_kernel<T><<<vblocks, pb::kThreads, 0, s>>>(                \
                static_cast<const T*>(grad_out), static_cast<const T*>(gate), static_cast<const T*>(up), \
                static_cast<T*>(grad_gate), static_cast<T*>(grad_up), nvec);             \
        if (done < n)                                                                    \
            pb::swiglu_bwd_kernel<T><<<blocks, pb::kThreads, 0, s>>>(                     \
                static_cast<const T*>(grad_out), static_cast<const T*>(gate), static_cast<const T*>(up), \
                static_cast<T*>(grad_gate), static_cast<T*>(grad_up), done, n);          \
    } while (0)
    switch (dtype) {
        case PARAS_F32: PB_BWD(float); break;
        case PARAS_BF16: PB_BWD(__nv_bfloat16); break;
        default: PB_BWD(__half); break;
    }
#undef PB_BWD
    PB_LAUNCH_CHECK("swiglu_bwd_kernel");
    return PARAS_OK;
}

int paras_b200_scale_columns(int gpu, const void* weight, const void* scale, void* out, int64_t N, int64_t K,
                             int dtype, void* stream) {
    if (N < 0 || K < 0) return fail(PARAS_E_INVALID, "paras scale_columns: negative size");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras scale_columns: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    const int64_t n = N * K;
    if (n == 0) return PARAS_OK;
    if (!weight || !scale || !out) return fail(PARAS_E_INVALID, "paras scale_columns: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    const int blocks = pb::grid_for(g, n, pb::kThreads);
#define PB_SCL(T)                                                                    \
    pb::scale_columns_kernel<T><<<blocks, pb::kThreads, 0, s>>>(                      \
        static_cast<const T*>(weight), static_cast<const T*>(scale), static_cast<T*>(out), n, K)
    switch (dtype) {
        case PARAS_F32: PB_SCL(float); break;
        case PARAS_BF16: PB_SCL(__nv_bfloat16); break;
        default: PB_SCL(__half); break;
    }
#undef PB_SCL
    PB_LAUNCH_CHECK("scale_columns_kernel");
    return PARAS_OK;
}

int paras_b200_rope(int gpu, const void* x, const int64_t* x_strides, const void* cosv, const void* sinv, void* out,
                    int B, int H, int L, int D, int64_t pos0, int dtype, void* stream) {
    if (B < 0 || H < 0 || L < 0 || D < 0 || pos0 < 0) return fail(PARAS_E_INVALID, "paras rope: negative size");
    if (D % 2) return fail(PARAS_E_INVALID, "paras rope: last dimension must be even");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras rope: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    const int64_t n = int64_t(B) * H * L * (D / 2);
    if (n == 0) return PARAS_OK;
    if (!x || !x_strides || !cosv || !sinv || !out) return fail(PARAS_E_INVALID, "paras rope: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    // 16-bit rows readable 16 bytes at a time (both halves): the vector kernel
    const bool vec = dtype != PARAS_F32 && D % 16 == 0 && x_strides[2] % 8 == 0 && x_strides[1] % 8 == 0 &&
                     x_strides[0] % 8 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv) |
                       reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (vec) {
        const int64_t units = int64_t(B) * H * L * (D / 16);
        const int vblocks = pb::grid_for(g, units, pb::kThreads);
        auto px = static_cast<const uint16_t*>(x);
        auto pc = static_cast<const uint16_t*>(cosv);
        auto ps = static_cast<const uint16_t*>(sinv);
        auto po = static_cast<uint16_t*>(out);
        if (dtype == PARAS_BF16)
            pb::rope_vec16_kernel<true><<<vblocks, pb::kThreads, 0, s>>>(px, pc, ps, po, units, H, L, D, x_strides[0], x_strides[1], x_strides[2], pos0);
        else
            pb::rope_vec16_kernel<false><<<vblocks, pb::kThreads, 0, s>>>(px, pc, ps, po, units, H, L, D, x_strides[0], x_strides[1], x_strides[2], pos0);
        PB_LAUNCH_CHECK("rope_vec16_kernel");
        return PARAS_OK;
    }
    const int blocks = pb::grid_for(g, n, pb::kThreads);
#define PB_ROPE(T)                                                                                   \
    pb::rope_kernel<T><<<blocks, pb::kThreads, 0, s>>>(                                               \
        static_cast<const T*>(x), static_cast<const T*>(cosv), static_cast<const T*>(sinv),          \
        static_cast<T*>(out), n, H, L, D, x_strides[0], x_strides[1], x_strides[2], pos0)
    switch (dtype) {
        case PARAS_F32: PB_ROPE(float); break;
        case PARAS_BF16: PB_ROPE(__nv_bfloat16); break;
        default: PB_ROPE(__half); break;
    }
#undef PB_ROPE
    PB_LAUNCH_CHECK("rope_kernel");
    return PARAS_OK;
}

int paras_b200_rotate_half(int gpu, const void* x, void* out, int64_t rows, int64_t D, int dtype,
                           int backward, void* stream) {
    if (rows < 0 || D < 0) return fail(PARAS_E_INVALID, "paras rotate_half: negative size");
    if (D % 2) return fail(PARAS_E_INVALID, "paras rotate_half: last dimension must be even");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras rotate_half: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    const int64_t n = rows * D;
    if (n == 0) return PARAS_OK;
    if (!x || !out) return fail(PARAS_E_INVALID, "paras rotate_half: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    const int64_t per = 16 / int64_t(pb::dtype_size(dtype));
    const bool vec = (D / 2) % per == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const int blocks = pb::grid_for(g, vec ? n / per : n, pb::kThreads, 16);
#define PB_ROT(T)                                                                   \
    do {                                                                            \
        if (vec)                                                                    \
            pb::rotate_half_vec_kernel<T><<<blocks, pb::kThreads, 0, s>>>(           \
                static_cast<const T*>(x), static_cast<T*>(out), n / per, int(D / 2 / per), backward); \
        else                                                                        \
            pb::rotate_half_kernel<T><<<blocks, pb::kThreads, 0, s>>>(               \
                static_cast<const T*>(x), static_cast<T*>(out), n, D, backward);    \
    } while (0)
    switch (dtype) {
        case PARAS_F32: PB_ROT(float); break;
        case PARAS_BF16: PB_ROT(__nv_bfloat16); break;
        default: PB_ROT(__half); break;
    }
#undef PB_ROT
    PB_LAUNCH_CHECK("rotate_half_kernel");
    return PARAS_OK;
}

int paras_b200_strided_copy(int gpu, void* dst, int dst_code, const int64_t* dst_strides,
                            const void* src, int src_code, const int64_t* src_strides,
                            const int64_t* sizes, int ndim, void* stream) {
    if (ndim < 0 || ndim > 8)
        return fail(PARAS_E_UNSUPPORTED, "paras copy: rank %d exceeds kernel limit 8", ndim);
    if (dst_code < 0 || dst_code > PARAS_SC_BOOL || src_code < 0 || src_code > PARAS_SC_BOOL)
        return fail(PARAS_E_UNSUPPORTED, "paras copy: unsupported element type");
    if (ndim > 0 && (!sizes || !dst_strides || !src_strides))
        return fail(PARAS_E_INVALID, "paras copy: null shape");
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    pb::CopySpec sp{};
    sp.ndim = ndim;
    int64_t n = 1;
    for (int d = 0; d < ndim; ++d) {
        if (sizes[d] < 0) return fail(PARAS_E_INVALID, "paras copy: negative size");
        sp.sizes[d] = sizes[d];
        sp.sstr[d] = src_strides[d];
        sp.dstr[d] = dst_strides[d];
        n *= sizes[d];
    }
    if (n == 0) return PARAS_OK;
    if (!dst || !src) return fail(PARAS_E_INVALID, "paras copy: null pointer");
    if (pb::copy_fast_path(g, dst, dst_code, src, src_code, sp, n, pb::pick_stream(g, stream))) {
        PB_LAUNCH_CHECK("copy fast path");
        return PARAS_OK;
    }
    const int blocks = pb::grid_for(g, n, pb::kThreads, 16);
    pb::strided_copy_kernel<<<blocks, pb::kThreads, 0, pb::pick_stream(g, stream)>>>(
        dst, dst_code, src, src_code, sp, n);
    PB_LAUNCH_CHECK("strided_copy_kernel");
    return PARAS_OK;
}

int paras_b200_fill(int gpu, void* dst, int code, double value, int64_t n, void* stream) {
    if (n < 0) return fail(PARAS_E_INVALID, "paras fill: negative element count");
    if (code < 0 || code > PARAS_SC_BOOL)
        return fail(PARAS_E_UNSUPPORTED, "paras fill: unsupported element type");
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (n == 0) return PARAS_OK;
    if (!dst) return fail(PARAS_E_INVALID, "paras fill: null pointer");
    const int blocks = pb::grid_for(g, n, pb::kThreads);
    pb::fill_kernel<<<blocks, pb::kThreads, 0, pb::pick_stream(g, stream)>>>(dst, code, value, n);
    PB_LAUNCH_CHECK("fill_kernel");
    return PARAS_OK;
}

}  // extern "C"
