// RMSNorm forward/backward for sm_100a.
//
// Replaces (a) the reference's fused paras::rms_norm lambda (csrc/ops/fused_ops.cpp:43-88:
// ONE THREAD per row, serial over H, double math, uncoalesced) and (b) the aten::rms_norm
// composite (csrc/ops/rms_swiglu_ops.cpp:43-75: pow, mean, add, rsqrt, mul, mul = six
// full passes over HBM, each rounding to the tensor dtype).
//
// Forward kernels: the whole row held in registers -- by one WARP for rows up to 128 vectors of
// 16 bytes, by a CTA of 4 or 8 warps for longer ones -- so HBM sees exactly one 128-bit
// coalesced read and one 128-bit write per element (algorithmic traffic
// 2*rows*H*sizeof(T) + H*sizeof(T)); sum of squares via warp shuffles, accumulated in
// double so that 16-bit results reproduce the reference's double arithmetic.  Rows too
// long for registers take a CTA-per-row two-pass kernel whose second read hits L2.
//
// MODE PARAS_ROUND_ONCE   : y = T((x * rstd) * w), rstd = 1/sqrt(sum(x^2)/H + eps)
// MODE PARAS_ROUND_PER_OP : emulates the composite's per-op rounding (pointwise_ops.cpp:
//                           33-52 unary, 62-85 binary, 246-249 mean = sum then *1/N).
#include "common.cuh"

namespace pb {
namespace {

constexpr int kWarpsPerBlock = 4;

template <typename T> struct RowMath {
    // value of x*x as the reference's pow(2) leaves it, plus its contribution to the sum
    template <int MODE> static __device__ __forceinline__ float sq(float x) {
        if constexpr (MODE == PARAS_ROUND_PER_OP) return round_to<T>(x * x);
        return x * x;
    }
};

// Per-row scalar pipeline shared by both kernels.  `ss` is the (double) sum of squares.
template <typename T, int MODE>
__device__ __forceinline__ void row_scalars(double ss, int64_t H, double eps, float* inv_f,
                                            double* inv_d) {
    if constexpr (MODE == PARAS_ROUND_ONCE) {
        const double r = 1.0 / sqrt(ss / double(H) + eps);
        *inv_d = r;
        *inv_f = float(r);
    } else {
        // sum -> T, *1/N -> T, +eps(T) -> T, rsqrt -> T ; each via double -> float -> T
        float s = round_to<T>(float(ss));
        s = round_to<T>(float(double(s) * (1.0 / double(H))));
        s = round_to<T>(float(double(s) + eps));
        s = round_to<T>(float(1.0 / sqrt(double(s))));
        *inv_f = s;
        *inv_d = double(s);
    }
}

template <typename T, int MODE>
__device__ __forceinline__ T finish(T xv, float inv_f, double inv_d, bool has_w, T wv) {
    if constexpr (MODE == PARAS_ROUND_ONCE) {
        if constexpr (sizeof(T) == 4) {
            double y = double(xv) * inv_d;
            if (has_w) y *= double(wv);
            return float(y);
        } else {
            float y = to_f32<T>(xv) * inv_f;
            if (has_w) y *= to_f32<T>(wv);
            return from_f32<T>(y);
        }
    } else {
        float y = round_to<T>(to_f32<T>(xv) * inv_f);
        if (has_w) y = round_to<T>(y * to_f32<T>(wv));
        return from_f32<T>(y);
    }
}

// Packed 16-bit arithmetic for the per-op-rounding mode: a bf16x2 / f16x2 multiply rounds
// its exact product once to the 16-bit type, which is precisely what "compute, then cast
// to the tensor dtype" means for a product of two 16-bit values -- at half an instruction
// per element instead of a convert/multiply/convert chain.
template <typename T> struct Packed;
template <> struct Packed<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ T2 dup(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ float2 unpack(T2 v) { return __bfloat1622float2(v); }
};
template <> struct Packed<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ T2 dup(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ float2 unpack(T2 v) { return __half22float2(v); }
};

// KV = 16-byte vectors per lane (row held in registers).  nvec = H / N vectors per row.
template <typename T, int MODE, int KV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, KV >= 16 ? 5 : 8)
rmsnorm_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                        float* __restrict__ rstd, int64_t rows, int64_t H, int nvec, double eps) {
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const T* xr = x + row * H;
        Vec16<T> v[KV];
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) v[k] = ld16_stream(xr + int64_t(i) * N);
        }
        double acc = 0.0;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) {
                if constexpr (sizeof(T) == 4) {
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        const float f = v[k].v[e];
                        acc += (MODE == PARAS_ROUND_ONCE) ? double(f) * double(f) : double(f * f);
                    }
                } else if constexpr (MODE == PARAS_ROUND_PER_OP) {
                    using T2 = typename Packed<T>::T2;
                    const T2* x2 = reinterpret_cast<const T2*>(&v[k]);
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < N / 2; ++e) {
                        const float2 f = Packed<T>::unpack(__hmul2(x2[e], x2[e]));  // pow(2), rounded
                        part += f.x + f.y;
                    }
                    acc += double(part);
                } else {
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < N; ++e)
                        part += RowMath<T>::template sq<MODE>(to_f32<T>(v[k].v[e]));
                    acc += double(part);
                }
            }
        }
        // Keep the row in its packed form across the reduction: without this fence the
        // compiler keeps the fp32 copies of all elements live as well (twice the registers,
        // a third of the occupancy).
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            uint4& u = *reinterpret_cast<uint4*>(&v[k]);
            asm volatile("" : "+r"(u.x), "+r"(u.y), "+r"(u.z), "+r"(u.w));
        }
        acc = warp_sum(acc);
        float inv_f;
        double inv_d;
        row_scalars<T, MODE>(acc, H, eps, &inv_f, &inv_d);
        if (rstd && lane == 0) rstd[row] = inv_f;
        T* yr = y + row * H;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = lane + 32 * k;
            if (i < nvec) {
                Vec16<T> wv;
                if (w) wv = ld16(w + int64_t(i) * N);
                Vec16<T> o;
                if constexpr (sizeof(T) == 2 && MODE == PARAS_ROUND_PER_OP) {
                    using T2 = typename Packed<T>::T2;
                    const T2 inv2 = Packed<T>::dup(inv_f);  // inv_f is already a value of T
                    const T2* x2 = reinterpret_cast<const T2*>(&v[k]);
                    const T2* w2 = reinterpret_cast<const T2*>(&wv);
                    T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
                    for (int e = 0; e < N / 2; ++e) {
                        T2 t = __hmul2(x2[e], inv2);       // x * inv, rounded
                        if (w) t = __hmul2(t, w2[e]);      // * weight, rounded
                        o2[e] = t;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < N; ++e)
                        o.v[e] = finish<T, MODE>(v[k].v[e], inv_f, inv_d, w != nullptr,
                                                 w ? wv.v[e] : v[k].v[e]);
                }
                st16_stream(yr + int64_t(i) * N, o);
            }
        }
    }
}

// One CTA of W warps per row, the row still held in registers (KV 16-byte vectors per thread).
// For long rows this is the better geometry: a warp that owns a whole 8 KB row alternates between
// a load phase, a reduction and a store phase with nothing in flight in between, and few such
// warps fit an SM; W warps sharing the row hold a quarter (W = 4) of it each, four times as many
// rows are resident per SM at the same registers, and the unit of the tail is one row.
// MINB (CTAs per SM the register allocation must allow) was measured on [16384, 4096] bf16 rows
// with W = 4: 10 gave 5.9 / 6.2 TB/s (single-rounding / per-op-rounding mode) where the compiler's
// own choice (8) gave 5.4 / 5.9 and 12 or more spilled.
template <typename T, int MODE, int KV, int W, int MINB>
__global__ void __launch_bounds__(32 * W, MINB)
rmsnorm_fwd_cta_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                       float* __restrict__ rstd, int64_t rows, int64_t H, int nvec, double eps) {
    constexpr int N = Vec16<T>::N;
    __shared__ double part_sum[2][W];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int flip = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
        const T* xr = x + row * H;
        Vec16<T> v[KV];
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = tid + 32 * W * k;
            if (i < nvec) v[k] = ld16_stream(xr + int64_t(i) * N);
        }
        double acc = 0.0;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = tid + 32 * W * k;
            if (i < nvec) {
                if constexpr (sizeof(T) == 4) {
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        const float f = v[k].v[e];
                        acc += (MODE == PARAS_ROUND_ONCE) ? double(f) * double(f) : double(f * f);
                    }
                } else if constexpr (MODE == PARAS_ROUND_PER_OP) {
                    using T2 = typename Packed<T>::T2;
                    const T2* x2 = reinterpret_cast<const T2*>(&v[k]);
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < N / 2; ++e) {
                        const float2 f = Packed<T>::unpack(__hmul2(x2[e], x2[e]));  // pow(2), rounded
                        part += f.x + f.y;
                    }
                    acc += double(part);
                } else {
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < N; ++e)
                        part += RowMath<T>::template sq<MODE>(to_f32<T>(v[k].v[e]));
                    acc += double(part);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < KV; ++k) {  // keep the row packed across the reduction (see above)
            uint4& u = *reinterpret_cast<uint4*>(&v[k]);
            asm volatile("" : "+r"(u.x), "+r"(u.y), "+r"(u.z), "+r"(u.w));
        }
        acc = warp_sum(acc);
        if (lane == 0) part_sum[flip][warp] = acc;
        __syncthreads();  // one barrier per row: the two sets of partials take turns
        double total = 0.0;
#pragma unroll
        for (int i = 0; i < W; ++i) total += part_sum[flip][i];
        float inv_f;
        double inv_d;
        row_scalars<T, MODE>(total, H, eps, &inv_f, &inv_d);
        if (rstd && tid == 0) rstd[row] = inv_f;
        T* yr = y + row * H;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int i = tid + 32 * W * k;
            if (i < nvec) {
                Vec16<T> wv;
                if (w) wv = ld16(w + int64_t(i) * N);
                Vec16<T> o;
                if constexpr (sizeof(T) == 2 && MODE == PARAS_ROUND_PER_OP) {
                    using T2 = typename Packed<T>::T2;
                    const T2 inv2 = Packed<T>::dup(inv_f);
                    const T2* x2 = reinterpret_cast<const T2*>(&v[k]);
                    const T2* w2 = reinterpret_cast<const T2*>(&wv);
                    T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
                    for (int e = 0; e < N / 2; ++e) {
                        T2 t = __hmul2(x2[e], inv2);
                        if (w) t = __hmul2(t, w2[e]);
                        o2[e] = t;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < N; ++e)
                        o.v[e] = finish<T, MODE>(v[k].v[e], inv_f, inv_d, w != nullptr,
                                                 w ? wv.v[e] : v[k].v[e]);
                }
                st16_stream(yr + int64_t(i) * N, o);
            }
        }
    }
}

// Any H, any alignment: one CTA per row, two passes (the second read is an L2 hit).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_block_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                         float* __restrict__ rstd, int64_t rows, int64_t H, double eps) {
    __shared__ double red[8];
    __shared__ double total;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * H;
        double acc = 0.0;
        for (int64_t j = threadIdx.x; j < H; j += blockDim.x) {
            const float f = to_f32<T>(xr[j]);
            if constexpr (sizeof(T) == 4 && MODE == PARAS_ROUND_ONCE)
                acc += double(f) * double(f);
            else
                acc += double(RowMath<T>::template sq<MODE>(f));
        }
        acc = warp_sum(acc);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int i = 0; i < int(blockDim.x >> 5); ++i) t += red[i];
            total = t;
        }
        __syncthreads();
        float inv_f;
        double inv_d;
        row_scalars<T, MODE>(total, H, eps, &inv_f, &inv_d);
        if (rstd && threadIdx.x == 0) rstd[row] = inv_f;
        T* yr = y + row * H;
        for (int64_t j = threadIdx.x; j < H; j += blockDim.x)
            yr[j] = finish<T, MODE>(xr[j], inv_f, inv_d, w != nullptr, w ? w[j] : xr[j]);
        __syncthreads();
    }
}

// rstd only (the statistic of paras::rms_norm, fused_ops.cpp:67-75): four warps per row, one read
// of x, no output tensor.  Feeds the row-scale epilogue of the GEMM.
template <typename T>
__global__ void __launch_bounds__(128)
rms_rstd_kernel(const T* __restrict__ x, float* __restrict__ rstd, int64_t rows, int64_t H, double eps, bool vec) {
    constexpr int N = Vec16<T>::N;
    __shared__ double part[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * H;
        double acc = 0.0;
        if (vec) {
            for (int64_t i = tid; i < H / N; i += 128) {
                const Vec16<T> v = ld16_stream(xr + i * N);
                float pf = 0.f;
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float f = to_f32<T>(v.v[e]);
                    if constexpr (sizeof(T) == 4) acc += double(f) * double(f);
                    else pf = fmaf(f, f, pf);
                }
                acc += double(pf);
            }
        } else {
            for (int64_t j = tid; j < H; j += 128) {
                const double f = to_f32<T>(xr[j]);
                acc += f * f;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) part[warp] = acc;
        __syncthreads();
        if (tid == 0) rstd[row] = float(1.0 / sqrt((part[0] + part[1] + part[2] + part[3]) / double(H) + eps));
        __syncthreads();
    }
}

// grad_x (fused_ops.cpp:111-135): one warp per row.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_bwd_dx_kernel(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ w,
                      const float* __restrict__ rstd, T* __restrict__ gx, int64_t rows, int64_t H) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const T* gr = go + row * H;
        const T* xr = x + row * H;
        double dot = 0.0;
        for (int64_t j = lane; j < H; j += 32)
            dot += double(to_f32<T>(gr[j])) * double(to_f32<T>(w[j])) * double(to_f32<T>(xr[j]));
        dot = warp_sum(dot);
        const double rr = double(rstd[row]);
        const double coef = rr * rr * rr / double(H);
        T* out = gx + row * H;
        for (int64_t j = lane; j < H; j += 32) {
            const double gj = to_f32<T>(gr[j]), wj = to_f32<T>(w[j]), xj = to_f32<T>(xr[j]);
            out[j] = from_f32<T>(float(gj * wj * rr - coef * xj * dot));
        }
    }
}

// grad_weight[j] = sum_r go[r,j]*x[r,j]*rstd[r] (fused_ops.cpp:137-155): a 32x32 thread
// tile per 32 columns, rows strided over the tile's second dimension.
template <typename T>
__global__ void __launch_bounds__(1024)
rmsnorm_bwd_dw_kernel(const T* __restrict__ go, const T* __restrict__ x,
                      const float* __restrict__ rstd, T* __restrict__ gw, int64_t rows, int64_t H) {
    __shared__ double part[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t col = int64_t(blockIdx.x) * 32 + tx;
    double acc = 0.0;
    if (col < H)
        for (int64_t r = ty; r < rows; r += 32)
            acc += double(to_f32<T>(go[r * H + col])) * double(to_f32<T>(x[r * H + col])) *
                   double(rstd[r]);
    part[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && col < H) {
        double t = 0.0;
        for (int i = 0; i < 32; ++i) t += part[i][tx];
        gw[col] = from_f32<T>(float(t));
    }
}

// Both gradients in one pass over grad_out and x (fused_ops.cpp:111-155): a CTA of THREADS threads takes
// whole rows, V 16-byte vectors per thread and tensor, so that a row's grad_out and x stay in registers
// between the row's dot product and its grad_x; each thread also keeps grad_weight partial sums for
// the columns it owns over all the rows its CTA walks.  The partials go to [gridDim.x, H] fp32 scratch
// that rmsnorm_bwd_dw_reduce_kernel sums (in double) and rounds.  HBM traffic: grad_out, x read once,
// grad_x written once.
template <typename T, int V, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_rows_kernel(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ w,
                        const float* __restrict__ rstd, T* __restrict__ gx, float* __restrict__ dw_part,
                        int64_t rows, int64_t H) {
    constexpr int N = Vec16<T>::N;
    __shared__ float red[2][THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    Vec16<T> wv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) wv[i] = ld16(w + (int64_t(tid) + int64_t(THREADS) * i) * N);
    float dwacc[V * N];
#pragma unroll
    for (int i = 0; i < V * N; ++i) dwacc[i] = 0.f;
    const float inv_h = 1.0f / float(H);
    int flip = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
        const T* gr = go + row * H;
        const T* xr = x + row * H;
        const float rr = rstd[row];   // asked for with the row: after the reduction it would be a round trip of its own
        Vec16<T> gv[V], xv[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            gv[i] = ld16_stream(gr + (int64_t(tid) + int64_t(THREADS) * i) * N);
            xv[i] = ld16_stream(xr + (int64_t(tid) + int64_t(THREADS) * i) * N);
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i)
#pragma unroll
            for (int e = 0; e < N; ++e)
                dot = fmaf(to_f32<T>(gv[i].v[e]) * to_f32<T>(wv[i].v[e]), to_f32<T>(xv[i].v[e]), dot);
        dot = warp_sum(dot);
        if (lane == 0) red[flip][warp] = dot;
        __syncthreads();          // (the buffer alternates: the next row's writes cannot overtake these reads)
        dot = 0.f;
#pragma unroll
        for (int i = 0; i < THREADS / 32; ++i) dot += red[flip][i];
        const float coef = rr * rr * rr * inv_h * dot;
        T* out = gx + row * H;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            Vec16<T> o;
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float g = to_f32<T>(gv[i].v[e]), xe = to_f32<T>(xv[i].v[e]);
                o.v[e] = from_f32<T>(fmaf(g * to_f32<T>(wv[i].v[e]), rr, -coef * xe));
                dwacc[i * N + e] = fmaf(g * xe, rr, dwacc[i * N + e]);
            }
            st16_stream(out + (int64_t(tid) + int64_t(THREADS) * i) * N, o);
        }
    }
    float* part = dw_part + int64_t(blockIdx.x) * H;
#pragma unroll
    for (int i = 0; i < V; ++i)
#pragma unroll
        for (int e = 0; e < N; e += 4)
            *reinterpret_cast<float4*>(part + (int64_t(tid) + int64_t(THREADS) * i) * N + e) =
                make_float4(dwacc[i * N + e], dwacc[i * N + e + 1], dwacc[i * N + e + 2], dwacc[i * N + e + 3]);
}

// The same with the rows arriving through a three-deep ring in shared memory (cp.async, 16 bytes per
// copy, each thread copying exactly the vectors it reads back, so the ring needs no barrier): the loads
// of the next two rows are in flight while a row is reduced and written.  The plain kernel above has a
// CTA's loads outstanding only between its store and its reduction, about half the time, and
// reaches 0.59 of the HBM peak at [16384, 4096]; bytes in flight are what it lacks.
constexpr int kBwdStages = 3;

// Registers a thread of the ring kernel needs, roughly: R rows of grad_out and x (V 16-byte vectors each),
// V*N grad_weight sums, the weight, and addressing.  Decides, on both sides of the launch, how many
// CTAs (one or two) share an SM.
// (An estimate on the generous side: a second CTA that squeezes the kernel into spills costs more than it
// brings: [16384, 4096] bf16 went from 0.074 to 0.161 ms under a bound of three CTAs.)
constexpr int bwd_regs(int v, int n, int r) { return 12 * v * r + v * n + 4 * v + 40; }
constexpr int bwd_ctas(int threads, int v, int n, int r) { return bwd_regs(v, n, r) * threads * 2 <= 65536 ? 2 : 1; }

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T, int V, int THREADS, int R, bool TAIL>
__global__ void __launch_bounds__(THREADS, bwd_ctas(THREADS, V, Vec16<T>::N, R))
rmsnorm_bwd_rows_pipe_kernel(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ w,
                             const float* __restrict__ rstd, T* __restrict__ gx, float* __restrict__ dw_part,
                             int64_t rows, int64_t H) {
    // A step is R consecutive rows: their reductions run side by side and share one barrier, which is
    // what a CTA's time per row mostly consists of once the loads are ahead.
    constexpr int N = Vec16<T>::N;
    extern __shared__ __align__(16) unsigned char ring_raw[];   // [stage][row of the step][go | x][THREADS * V] vectors
    __shared__ float red[2][R][THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_raw));
    constexpr uint32_t kHalf = THREADS * V * 16, kRow = 2 * kHalf, kStage = R * kRow;
    const int64_t steps = (rows + R - 1) / R;
    // V = ceil(vectors per row / THREADS): only a thread's last vector can lie past the end of the row, and
    // only in the TAIL instantiation (its own: the checks cost the kernel that sits at the register limit 12 %)
    const bool last_ok = !TAIL || int64_t(tid) + int64_t(THREADS) * (V - 1) < H / N;
    Vec16<T> zero;
#pragma unroll
    for (int e = 0; e < N; ++e) zero.v[e] = from_f32<T>(0.f);
    auto issue = [&](int64_t step, int stage) {
        if (step < steps) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int64_t row = step * R + r;
                if (row < rows) {
                    const T* gr = go + row * H;
                    const T* xr = x + row * H;
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        if (i == V - 1 && !last_ok) break;
                        const uint32_t off = (uint32_t(tid) + uint32_t(THREADS) * i) * 16;
                        cp_async16(ring + stage * kStage + r * kRow + off, gr + (int64_t(tid) + int64_t(THREADS) * i) * N);
                        cp_async16(ring + stage * kStage + r * kRow + kHalf + off, xr + (int64_t(tid) + int64_t(THREADS) * i) * N);
                    }
                }
            }
        }
        cp_async_commit();   // an empty group past the last step keeps the group count uniform
    };
    Vec16<T> wv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) wv[i] = (i < V - 1 || last_ok) ? ld16(w + (int64_t(tid) + int64_t(THREADS) * i) * N) : zero;
    float dwacc[V * N];
#pragma unroll
    for (int i = 0; i < V * N; ++i) dwacc[i] = 0.f;
    const float inv_h = 1.0f / float(H);
#pragma unroll
    for (int st = 0; st < kBwdStages - 1; ++st) issue(int64_t(blockIdx.x) + int64_t(st) * gridDim.x, st);
    int flip = 0, stage = 0;
    float rr_next[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rr_next[r] = rstd[min(int64_t(blockIdx.x) * R + r, rows - 1)];
    for (int64_t step = blockIdx.x; step < steps; step += gridDim.x, flip ^= 1) {
        // the stage refilled here is the one this thread emptied in the previous iteration
        issue(step + int64_t(kBwdStages - 1) * gridDim.x, stage == 0 ? kBwdStages - 1 : stage - 1);
        float rr[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            rr[r] = rr_next[r];   // a scalar miss of its own: asked for a step ahead
            rr_next[r] = rstd[min((step + gridDim.x) * R + r, rows - 1)];
        }
        cp_async_wait<kBwdStages - 1>();
        Vec16<T> gv[R][V], xv[R][V];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const uint32_t off = (uint32_t(tid) + uint32_t(THREADS) * i) * 16;
                gv[r][i] = *reinterpret_cast<const Vec16<T>*>(ring_raw + stage * kStage + r * kRow + off);
                xv[r][i] = *reinterpret_cast<const Vec16<T>*>(ring_raw + stage * kStage + r * kRow + kHalf + off);
                if (i == V - 1 && !last_ok) gv[r][i] = xv[r][i] = zero;   // nothing was copied there
            }
        stage = stage + 1 == kBwdStages ? 0 : stage + 1;
        float dot[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            dot[r] = 0.f;
#pragma unroll
            for (int i = 0; i < V; ++i)
#pragma unroll
                for (int e = 0; e < N; ++e)
                    dot[r] = fmaf(to_f32<T>(gv[r][i].v[e]) * to_f32<T>(wv[i].v[e]), to_f32<T>(xv[r][i].v[e]), dot[r]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < R; ++r) dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], o);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) red[flip][r][warp] = dot[r];
        }
        __syncthreads();          // (the buffer alternates: the next step's writes cannot overtake these reads)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int64_t row = step * R + r;
            if (row >= rows) break;   // the same for every thread; rows past the end hold stale ring data
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < THREADS / 32; ++i) d += red[flip][r][i];
            const float coef = rr[r] * rr[r] * rr[r] * inv_h * d;
            T* out = gx + row * H;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                Vec16<T> o;
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float g = to_f32<T>(gv[r][i].v[e]), xe = to_f32<T>(xv[r][i].v[e]);
                    o.v[e] = from_f32<T>(fmaf(g * to_f32<T>(wv[i].v[e]), rr[r], -coef * xe));
                    dwacc[i * N + e] = fmaf(g * xe, rr[r], dwacc[i * N + e]);
                }
                if (i < V - 1 || last_ok) st16_stream(out + (int64_t(tid) + int64_t(THREADS) * i) * N, o);
            }
        }
    }
    cp_async_wait<0>();
    float* part = dw_part + int64_t(blockIdx.x) * H;
#pragma unroll
    for (int i = 0; i < V; ++i)
#pragma unroll
        for (int e = 0; e < N; e += 4)
            if (i < V - 1 || last_ok) *reinterpret_cast<float4*>(part + (int64_t(tid) + int64_t(THREADS) * i) * N + e) =
                make_float4(dwacc[i * N + e], dwacc[i * N + e + 1], dwacc[i * N + e + 2], dwacc[i * N + e + 3]);
}

// grad_weight[j] = sum over the partial rows: 32 threads per column take every thirty-second partial
// (H / 32 CTAs: at H = 4096 that is 128 of them, and a thread's chain of loads is 5-10 long).
template <typename T>
__global__ void __launch_bounds__(1024)
rmsnorm_bwd_dw_reduce_kernel(const float* __restrict__ dw_part, T* __restrict__ gw, int parts, int64_t H) {
    __shared__ double sh[32][33];
    const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
    const int64_t col = int64_t(blockIdx.x) * 32 + cx;
    double acc = 0.0;
    if (col < H) {
#pragma unroll 4
        for (int pi = py; pi < parts; pi += 32) acc += double(__ldcs(dw_part + int64_t(pi) * H + col));
    }
    sh[py][cx] = acc;
    __syncthreads();
    if (py == 0 && col < H) {
        double t = 0.0;
#pragma unroll
        for (int i = 0; i < 32; ++i) t += sh[i][cx];
        gw[col] = from_f32<T>(float(t));
    }
}

struct BwdRowsArgs {
    const void *go, *x, *w;
    const float* rstd;
    void* gx;
    float* part;
    int64_t rows, H;
    int parts;
    bool pipe, tail;
    int rstep;
    size_t ring;
    cudaStream_t s;
};

template <typename T, int V, int THREADS, int R, bool TAIL = false>
void launch_bwd_pipe(const BwdRowsArgs& a) {
    cudaFuncSetAttribute(rmsnorm_bwd_rows_pipe_kernel<T, V, THREADS, R, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(a.ring));
    rmsnorm_bwd_rows_pipe_kernel<T, V, THREADS, R, TAIL><<<a.parts, THREADS, a.ring, a.s>>>(
        static_cast<const T*>(a.go), static_cast<const T*>(a.x), static_cast<const T*>(a.w), a.rstd, static_cast<T*>(a.gx),
        a.part, a.rows, a.H);
}

template <typename T, int V, int THREADS>
void launch_bwd_rows(const BwdRowsArgs& a) {
    if (a.pipe) {
        if (a.tail) return launch_bwd_pipe<T, V, THREADS, 1, true>(a);
        if constexpr (V <= 2) {
            if (a.rstep == 4) return launch_bwd_pipe<T, V, THREADS, 4>(a);
        }
        if constexpr (V <= 4) {
            if (a.rstep == 2) return launch_bwd_pipe<T, V, THREADS, 2>(a);
        }
        return launch_bwd_pipe<T, V, THREADS, 1>(a);
    }
    rmsnorm_bwd_rows_kernel<T, V, THREADS><<<a.parts, THREADS, 0, a.s>>>(
        static_cast<const T*>(a.go), static_cast<const T*>(a.x), static_cast<const T*>(a.w), a.rstd, static_cast<T*>(a.gx),
        a.part, a.rows, a.H);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

double round_scalar_to(double v, int dtype) {
    // what wrapping a scalar into a 0-dim tensor of the output dtype does (double->float->T)
    float f = float(v);
    if (dtype == PARAS_BF16) return double(__bfloat162float(__float2bfloat16_rn(f)));
    if (dtype == PARAS_F16) return double(__half2float(__float2half_rn(f)));
    return double(f);
}

template <typename T, int MODE>
int launch_fwd(Gpu* g, const void* x, const void* w, void* y, float* rstd, int64_t rows,
               int64_t H, double eps, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    const T* px = static_cast<const T*>(x);
    const T* pw = static_cast<const T*>(w);
    T* py = static_cast<T*>(y);
    const bool vec_ok = (H % N == 0) && aligned16(x) && aligned16(y) && (!w || aligned16(w));
    const int64_t nvec = H / N;
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    if (vec_ok && nvec > 32 * 4 && nvec <= 32 * 8 * 4) {
        // long rows: W warps share a row, 4 vectors per thread (4 warps up to 8 KB rows, else 8)
        int64_t blocks = rows;
        const int64_t cap = int64_t(1) << 30;
        if (blocks > cap) blocks = cap;
        if (nvec <= 32 * 4 * 4)
            rmsnorm_fwd_cta_kernel<T, MODE, 4, 4, 10><<<int(blocks), 128, 0, s>>>(px, pw, py, rstd, rows, H, int(nvec), eps);
        else
            rmsnorm_fwd_cta_kernel<T, MODE, 4, 8, 5><<<int(blocks), 256, 0, s>>>(px, pw, py, rstd, rows, H, int(nvec), eps);
        PB_LAUNCH_CHECK("rmsnorm_fwd_cta_kernel");
        return PARAS_OK;
    }
    if (vec_ok && nvec <= 32 * 16) {
        // One row per warp and as many small CTAs as there are row groups: the block scheduler
        // balances them, and every resident warp keeps a whole row (up to 8 KB) in flight.
        int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
        const int64_t cap = int64_t(1) << 30;
        if (blocks > cap) blocks = cap;
        const int kv = int((nvec + 31) / 32);
#define PB_RMS_LAUNCH(KV)                                                                   \
    rmsnorm_fwd_warp_kernel<T, MODE, KV><<<int(blocks), kWarpsPerBlock * 32, 0, s>>>(        \
        px, pw, py, rstd, rows, H, int(nvec), eps)
        if (kv <= 1) PB_RMS_LAUNCH(1);
        else if (kv <= 2) PB_RMS_LAUNCH(2);
        else if (kv <= 4) PB_RMS_LAUNCH(4);
        else if (kv <= 8) PB_RMS_LAUNCH(8);
        else PB_RMS_LAUNCH(16);
#undef PB_RMS_LAUNCH
        PB_LAUNCH_CHECK("rmsnorm_fwd_warp_kernel");
        return PARAS_OK;
    }
    int64_t blocks = rows;
    const int64_t cap = int64_t(sms) * 8;
    if (blocks > cap) blocks = cap;
    rmsnorm_fwd_block_kernel<T, MODE><<<int(blocks), 256, 0, s>>>(px, pw, py, rstd, rows, H, eps);
    PB_LAUNCH_CHECK("rmsnorm_fwd_block_kernel");
    return PARAS_OK;
}

}  // namespace
}  // namespace pb

using pb::fail;
using pb::Gpu;

extern "C" {

int paras_b200_rmsnorm_fwd(int gpu, const void* x, const void* weight, void* y, float* rstd,
                           int64_t rows, int64_t H, double eps, int dtype, int mode,
                           void* stream) {
    pb::NvtxRange range("paras_b200_rmsnorm_fwd");
    if (rows < 0 || H < 0) return fail(PARAS_E_INVALID, "paras rms_norm: negative size");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras rms_norm: unsupported dtype %d", dtype);
    if (mode != PARAS_ROUND_ONCE && mode != PARAS_ROUND_PER_OP)
        return fail(PARAS_E_INVALID, "paras rms_norm: bad rounding mode %d", mode);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (rows == 0 || H == 0) return PARAS_OK;
    if (!x || !y) return fail(PARAS_E_INVALID, "paras rms_norm: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    const double eps_used = mode == PARAS_ROUND_PER_OP ? pb::round_scalar_to(eps, dtype) : eps;
#define PB_RMS(T)                                                                            \
    (mode == PARAS_ROUND_ONCE                                                                \
         ? pb::launch_fwd<T, PARAS_ROUND_ONCE>(g, x, weight, y, rstd, rows, H, eps_used, s)  \
         : pb::launch_fwd<T, PARAS_ROUND_PER_OP>(g, x, weight, y, rstd, rows, H, eps_used, s))
    switch (dtype) {
        case PARAS_F32: return PB_RMS(float);
        case PARAS_BF16: return PB_RMS(__nv_bfloat16);
        default: return PB_RMS(__half);
    }
#undef PB_RMS
}

int paras_b200_rms_rstd(int gpu, const void* x, float* rstd, int64_t rows, int64_t H, double eps, int dtype,
                        void* stream) {
    if (rows < 0 || H < 0) return fail(PARAS_E_INVALID, "paras rms_rstd: negative size");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras rms_rstd: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (rows == 0) return PARAS_OK;
    if (H == 0 || !x || !rstd) return fail(PARAS_E_INVALID, "paras rms_rstd: null pointer or empty rows");
    cudaStream_t s = pb::pick_stream(g, stream);
    const int64_t cap = int64_t(1) << 30;
    const int blocks = int(rows < cap ? rows : cap);
    const size_t es = pb::dtype_size(dtype);
    const bool vec = pb::aligned16(x) && (size_t(H) * es) % 16 == 0;
    switch (dtype) {
        case PARAS_F32: pb::rms_rstd_kernel<float><<<blocks, 128, 0, s>>>(static_cast<const float*>(x), rstd, rows, H, eps, vec); break;
        case PARAS_BF16: pb::rms_rstd_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rstd, rows, H, eps, vec); break;
        default: pb::rms_rstd_kernel<__half><<<blocks, 128, 0, s>>>(static_cast<const __half*>(x), rstd, rows, H, eps, vec); break;
    }
    PB_LAUNCH_CHECK("rms_rstd_kernel");
    return PARAS_OK;
}

int paras_b200_rmsnorm_bwd(int gpu, const void* grad_out, const void* x, const void* weight,
                           const float* rstd, void* grad_x, void* grad_weight, int64_t rows,
                           int64_t H, int dtype, void* stream) {
    pb::NvtxRange range("paras_b200_rmsnorm_bwd");
    if (rows < 0 || H < 0) return fail(PARAS_E_INVALID, "paras rms_norm_backward: negative size");
    if (dtype != PARAS_F32 && dtype != PARAS_BF16 && dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras rms_norm_backward: unsupported dtype %d", dtype);
    int st;
    Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (H == 0) return PARAS_OK;
    if (!grad_weight) return fail(PARAS_E_INVALID, "paras rms_norm_backward: null pointer");
    cudaStream_t s = pb::pick_stream(g, stream);
    if (rows == 0) {
        PB_CUDA(cudaMemsetAsync(grad_weight, 0, size_t(H) * pb::dtype_size(dtype), s));
        return PARAS_OK;
    }
    if (!grad_out || !x || !weight || !rstd || !grad_x)
        return fail(PARAS_E_INVALID, "paras rms_norm_backward: null pointer");
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    // Rows that split into 1..8 vectors per thread of a 128- or 256-thread CTA take the one-pass kernel.
    {
        const int64_t nvec = H * int64_t(pb::dtype_size(dtype)) / 16;
        const bool vec_ok = (H * int64_t(pb::dtype_size(dtype))) % 16 == 0 && pb::aligned16(grad_out) && pb::aligned16(x) &&
                            pb::aligned16(weight) && pb::aligned16(grad_x);
        // CTA size by row length, so that a thread holds at most 4 (last resort 8) vectors of a row; the ring
        // kernel takes rows that do not fill the last vector slot of every thread
        int threads = 0;
        if (vec_ok) threads = nvec <= 512 ? 128 : nvec <= 1024 ? 256 : nvec <= 4096 ? 512 : 0;
        if (threads) {
            const int v = int((nvec + threads - 1) / threads);
            // The ring variant: three stages of 1, 2 or 4 rows (grad_out and x) in shared memory, one or two
            // CTAs per SM as registers and shared memory allow.  Measured at [16384, 4096] bf16: 0.104 ms
            // without the ring, 0.085 with four CTAs per SM and one row per step, 0.074-0.076 with two CTAs
            // and two rows per step (fewer partial rows of grad_weight as well).
            const int nper = int(16 / pb::dtype_size(dtype));
            const size_t slot_bytes = size_t(threads) * v * 16;   // a row in the ring
            int rstep = 0, pipe_ctas = 1;
            const bool tail = nvec % threads != 0;
            for (int r = tail ? 1 : 4; r >= 1 && !rstep; r >>= 1) {
                if ((r == 4 && v > 2) || (r == 2 && v > 4)) continue;   // (not instantiated: too many registers)
                if (pb::bwd_regs(v, nper, r) * threads > 65536) continue;
                int ctas = pb::bwd_ctas(threads, v, nper, r);
                const size_t per_cta = size_t(pb::kBwdStages) * 2 * slot_bytes * r;
                while (ctas > 1 && per_cta * ctas > 200 * 1024) --ctas;
                if (per_cta * ctas <= 200 * 1024) { rstep = r; pipe_ctas = ctas; }
            }
            const size_t ring = size_t(pb::kBwdStages) * 2 * slot_bytes * (rstep ? rstep : 1);
            const bool pipe = rstep && rows >= int64_t(sms) * pipe_ctas * rstep;
            if (pipe || nvec % threads == 0) {   // (the plain one-pass kernel wants full slots)
            const int parts = int(std::min<int64_t>(rows, int64_t(sms) * (pipe ? pipe_ctas : threads == 128 ? 4 : threads == 256 ? 2 : 1)));
            void* scratch = nullptr;
            st = paras_b200_malloc_async(gpu, size_t(parts) * size_t(H) * sizeof(float), s, &scratch);
            if (st != PARAS_OK) return st;
            float* part = static_cast<float*>(scratch);
            const pb::BwdRowsArgs ra{grad_out, x, weight, rstd, grad_x, part, rows, H, parts, pipe, tail, rstep, ring, s};
#define PB_ROWS_V(T, TH)                                                                                         \
    switch (v) {                                                                                                 \
        case 1: pb::launch_bwd_rows<T, 1, TH>(ra); break; case 2: pb::launch_bwd_rows<T, 2, TH>(ra); break;       \
        case 3: pb::launch_bwd_rows<T, 3, TH>(ra); break; case 4: pb::launch_bwd_rows<T, 4, TH>(ra); break;       \
        case 5: pb::launch_bwd_rows<T, 5, TH>(ra); break; case 6: pb::launch_bwd_rows<T, 6, TH>(ra); break;       \
        case 7: pb::launch_bwd_rows<T, 7, TH>(ra); break; default: pb::launch_bwd_rows<T, 8, TH>(ra); break;      \
    }
#define PB_ROWS_T(T)                                                                                             \
    do {                                                                                                         \
        if (threads == 128) { PB_ROWS_V(T, 128) } else if (threads == 256) { PB_ROWS_V(T, 256) } else { PB_ROWS_V(T, 512) } \
        pb::rmsnorm_bwd_dw_reduce_kernel<T><<<int((H + 31) / 32), 1024, 0, s>>>(part, static_cast<T*>(grad_weight), parts, H); \
    } while (0)
            switch (dtype) {
                case PARAS_F32: PB_ROWS_T(float); break;
                case PARAS_BF16: PB_ROWS_T(__nv_bfloat16); break;
                default: PB_ROWS_T(__half); break;
            }
#undef PB_ROWS_T
#undef PB_ROWS_V
            st = cudaGetLastError() == cudaSuccess ? PARAS_OK : fail(PARAS_E_CUDA, "paras rms_norm_backward: kernel launch failed");
            const int st2 = paras_b200_free_async(gpu, scratch, s);
            return st != PARAS_OK ? st : st2;
            }
        }
    }
    int64_t blocks = (rows + pb::kWarpsPerBlock - 1) / pb::kWarpsPerBlock;
    if (blocks > int64_t(sms) * 16) blocks = int64_t(sms) * 16;
    const int dwblocks = int((H + 31) / 32);
#define PB_BWD(T)                                                                             \
    do {                                                                                      \
        pb::rmsnorm_bwd_dx_kernel<T><<<int(blocks), pb::kWarpsPerBlock * 32, 0, s>>>(          \
            static_cast<const T*>(grad_out), static_cast<const T*>(x),                        \
            static_cast<const T*>(weight), rstd, static_cast<T*>(grad_x), rows, H);           \
        pb::rmsnorm_bwd_dw_kernel<T><<<dwblocks, 1024, 0, s>>>(                               \
            static_cast<const T*>(grad_out), static_cast<const T*>(x), rstd,                  \
            static_cast<T*>(grad_weight), rows, H);                                           \
    } while (0)
    switch (dtype) {
        case PARAS_F32: PB_BWD(float); break;
        case PARAS_BF16: PB_BWD(__nv_bfloat16); break;
        default: PB_BWD(__half); break;
    }
#undef PB_BWD
    PB_LAUNCH_CHECK("rmsnorm_bwd kernels");
    return PARAS_OK;
}

}  // extern "C"
