/* Plain-C restatement of the reference's host-engine arithmetic for the transformer hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  The product never links or loads this file: tests/ load the
 * shared object built from it (make -C oracle cport) through ctypes and hold it, bit for bit,
 * to the golden vectors the unmodified reference produced (tests/golden/), next to the torch
 * restatement in oracle/oracle.py.  It exists so that the oracle does not rest on torch's CPU
 * kernels alone: every rounding step below is written out.
 *
 * Reference code restated (paths inside the reference project):
 *   csrc/ops/fused_ops.cpp:43-88      paras::rms_norm          double math, one rounding, rstd in fp32
 *   csrc/ops/fused_ops.cpp:90-157     paras::rms_norm_backward
 *   csrc/ops/fused_ops.cpp:162-194    paras::swiglu            g / (1 + exp(-g)) * u
 *   csrc/ops/fused_ops.cpp:196-229    paras::swiglu_backward
 *   csrc/ops/fused_ops.cpp:234-302    paras::rotate_half and its backward
 *   csrc/ops/rms_swiglu_ops.cpp:43-75 aten::rms_norm composite: pow, sum, *1/N, +eps, rsqrt, *inv,
 *                                     *weight, each rounded to the tensor dtype
 *   csrc/ops/rms_swiglu_ops.cpp:83-86 torch_paras::swiglu(x, gate) = x * silu(gate), silu rounded
 *   csrc/ops/pointwise_ops.cpp:926-981 softmax over the last dim: max, sum of exp, divide, in double
 *   csrc/ops/attention_ops.cpp:71-136 sdpa_math: scores = (q k^T) * scale, mask, softmax, @ v, every
 *                                     intermediate in the tensor dtype
 *
 * Storage types: 0 = float32, 1 = bfloat16, 2 = float16 (raw bits in uint16_t for the 16-bit
 * ones).  The reference's kernels read an element as double and write static_cast<scalar_t>(double),
 * which for the 16-bit types goes double -> float -> 16 bits (two roundings); store() does the same.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { PO_F32 = 0, PO_BF16 = 1, PO_F16 = 2 };

/* ---------------------------------------------------------------- 16-bit conversions */
static float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* round to nearest even; NaN stays a quiet NaN */
static uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0x1fu) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        /* subnormal: value = man * 2^-24 */
        const float v = (float)man * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static uint16_t f32_to_f16(float f) {
    const uint32_t u = f32_to_bits(f);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);         /* rounds to infinity (>= 65520) */
    if (a < 0x38800000u) {                                           /* below 2^-14: subnormal half */
        /* value * 2^24 rounded to nearest even gives the 10-bit mantissa (may carry into exp 1) */
        const float scaled = bits_to_f32(a) * 16777216.0f;           /* exact: power of two */
        const float r = nearbyintf(scaled);                          /* current mode: to nearest even */
        return (uint16_t)(sign | (uint16_t)r);
    }
    uint32_t v = a - 0x38000000u;                                    /* rebias 127 -> 15 */
    v += 0xfffu + ((v >> 13) & 1u);                                  /* nearest even on 13 dropped bits */
    return (uint16_t)(sign | (uint16_t)(v >> 13));
}

/* ---------------------------------------------------------------- typed element access */
static double load(const void* p, int64_t i, int dt) {
    switch (dt) {
        case PO_F32: return (double)((const float*)p)[i];
        case PO_BF16: return (double)bf16_to_f32(((const uint16_t*)p)[i]);
        default: return (double)f16_to_f32(((const uint16_t*)p)[i]);
    }
}

static void store(void* p, int64_t i, int dt, double v) {
    const float f = (float)v;
    switch (dt) {
        case PO_F32: ((float*)p)[i] = f; break;
        case PO_BF16: ((uint16_t*)p)[i] = f32_to_bf16(f); break;
        default: ((uint16_t*)p)[i] = f32_to_f16(f); break;
    }
}

/* v rounded to the storage type and read back, as when a kernel's output feeds the next kernel */
static double rounded(double v, int dt) {
    const float f = (float)v;
    switch (dt) {
        case PO_F32: return (double)f;
        case PO_BF16: return (double)bf16_to_f32(f32_to_bf16(f));
        default: return (double)f16_to_f32(f32_to_f16(f));
    }
}

static size_t elem_size(int dt) { return dt == PO_F32 ? 4 : 2; }

/* exported for the tests of the conversions themselves */
uint16_t po_f32_to_bf16(float f) { return f32_to_bf16(f); }
uint16_t po_f32_to_f16(float f) { return f32_to_f16(f); }
float po_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
float po_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* ---------------------------------------------------------------- paras::rms_norm (fused) */
/* fused_ops.cpp:43-88: per row, sum of squares in double left to right, rstd = 1/sqrt(ss/H + eps),
 * out = (x * rstd) * w rounded once; rstd is also returned as float. */
void po_rms_norm_fused(const void* x, const void* w, void* out, float* rstd, int64_t rows, int64_t h,
                       double eps, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int64_t i = 0; i < h; ++i) {
            const double v = load(x, r * h + i, dt);
            ss += v * v;
        }
        const double rms = 1.0 / sqrt(ss / (double)h + eps);
        if (rstd) rstd[r] = (float)rms;
        for (int64_t i = 0; i < h; ++i)
            store(out, r * h + i, dt, (load(x, r * h + i, dt) * rms) * load(w, i, dt));
    }
}

/* fused_ops.cpp:90-157: grad_in = g*w*rstd - rstd^3/H * x * sum(g*w*x); grad_w = column sums of
 * g*x*rstd taken row after row in double. */
void po_rms_norm_fused_backward(const void* g, const void* x, const void* w, const float* rstd,
                                void* grad_in, void* grad_w, int64_t rows, int64_t h, int dt, int wdt) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const double rr = (double)rstd[r];
        double dot = 0.0;
        for (int64_t i = 0; i < h; ++i)
            dot += load(g, r * h + i, dt) * load(w, i, wdt) * load(x, r * h + i, dt);
        const double coef = rr * rr * rr / (double)h;
        for (int64_t i = 0; i < h; ++i) {
            const double gi = load(g, r * h + i, dt), xi = load(x, r * h + i, dt);
            store(grad_in, r * h + i, dt, gi * load(w, i, wdt) * rr - coef * xi * dot);
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < h; ++i) {
        double acc = 0.0;
        for (int64_t r = 0; r < rows; ++r)
            acc += load(g, r * h + i, dt) * load(x, r * h + i, dt) * (double)rstd[r];
        store(grad_w, i, wdt, acc);
    }
}

/* ---------------------------------------------------------------- aten::rms_norm (composite) */
/* rms_swiglu_ops.cpp:43-75: x.pow(2) | sum over the normalised dims | * (1/N) | + eps | rsqrt |
 * x * inv | * weight -- each a kernel of its own that rounds to the tensor dtype; the scalars
 * (eps) are first materialised in that dtype (pointwise_ops.cpp:54-59).  w may be NULL. */
void po_rms_norm_composite(const void* x, const void* w, void* out, int64_t rows, int64_t n,
                           double eps, int dt) {
    const double eps_dt = rounded(eps, dt);
    const double inv_n = 1.0 / (double)n;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double ssum = 0.0;
        for (int64_t i = 0; i < n; ++i) {
            const double v = load(x, r * n + i, dt);
            ssum += rounded(pow(v, 2.0), dt);
        }
        double mean = rounded(ssum, dt);
        mean = rounded(mean * inv_n, dt);
        mean = rounded(mean + eps_dt, dt);
        const double inv = rounded(1.0 / sqrt(mean), dt);
        for (int64_t i = 0; i < n; ++i) {
            double o = rounded(load(x, r * n + i, dt) * inv, dt);
            if (w) o = rounded(o * load(w, i, dt), dt);
            store(out, r * n + i, dt, o);
        }
    }
}

/* ---------------------------------------------------------------- SwiGLU */
/* fused_ops.cpp:162-194 */
void po_swiglu_fused(const void* gate, const void* up, void* out, int64_t n, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double g = load(gate, i, dt);
        store(out, i, dt, (g / (1.0 + exp(-g))) * load(up, i, dt));
    }
}

/* fused_ops.cpp:196-229 */
void po_swiglu_fused_backward(const void* dy, const void* gate, const void* up, void* dgate, void* dup,
                              int64_t n, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double d = load(dy, i, dt), g = load(gate, i, dt), u = load(up, i, dt);
        const double s = 1.0 / (1.0 + exp(-g));
        store(dgate, i, dt, d * u * (s * (1.0 + g * (1.0 - s))));
        store(dup, i, dt, d * g * s);
    }
}

/* rms_swiglu_ops.cpp:83-86 with silu of pointwise_ops.cpp:460-464: silu(gate) is a kernel of its
 * own and rounds before the multiply. */
void po_swiglu_composite(const void* x, const void* gate, void* out, int64_t n, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double g = load(gate, i, dt);
        const double silu = rounded(g / (1.0 + exp(-g)), dt);
        store(out, i, dt, load(x, i, dt) * silu);
    }
}

/* ---------------------------------------------------------------- rotate_half */
/* fused_ops.cpp:234-267: out = cat(-x[d/2:], x[:d/2]); backward (269-302) = cat(g[d/2:], -g[:d/2]).
 * Negation is exact in every storage type, so bits are moved with the sign flipped. */
static void rotate(const void* x, void* out, int64_t rows, int64_t d, int dt, int backward) {
    const int64_t half = d / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < half; ++i) {
            const double lo = load(x, r * d + i, dt), hi = load(x, r * d + half + i, dt);
            store(out, r * d + i, dt, backward ? hi : -hi);
            store(out, r * d + half + i, dt, backward ? -lo : lo);
        }
}
int po_rotate_half(const void* x, void* out, int64_t rows, int64_t d, int dt) {
    if (d % 2) return 1;
    rotate(x, out, rows, d, dt, 0);
    return 0;
}
int po_rotate_half_backward(const void* g, void* out, int64_t rows, int64_t d, int dt) {
    if (d % 2) return 1;
    rotate(g, out, rows, d, dt, 1);
    return 0;
}

/* ---------------------------------------------------------------- softmax over the last dim */
/* pointwise_ops.cpp:954-977: per row the maximum, then the sum of exp(x - max) left to right, then
 * exp(x - max) / sum, all in double; one rounding on store.  A row of -inf only gives NaN
 * (exp(-inf - -inf)), as in the reference. */
static void softmax_row(const void* x, void* out, int64_t r, int64_t n, int dt) {
    double m = -INFINITY;
    for (int64_t i = 0; i < n; ++i) {
        const double v = load(x, r * n + i, dt);
        if (v > m) m = v;
    }
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += exp(load(x, r * n + i, dt) - m);
    for (int64_t i = 0; i < n; ++i) store(out, r * n + i, dt, exp(load(x, r * n + i, dt) - m) / s);
}

void po_softmax_lastdim(const void* x, void* out, int64_t rows, int64_t n, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) softmax_row(x, out, r, n, dt);
}

/* ---------------------------------------------------------------- scaled dot product attention */
/* attention_ops.cpp:71-136 for contiguous [B, Hq, Lq, D] queries and [B, Hkv, Lk, D] keys and values
 * (Hq a multiple of Hkv: query head h reads kv head h / (Hq/Hkv), which is what repeat_interleave
 * over the head dim gives, lines 82-92).  Steps, each leaving a tensor of the storage type:
 *   1. scores = q k^T                 the reference runs libtorch's CPU bmm on host copies
 *                                     (vision_ops.cpp:398-406); restated as a float accumulation over
 *                                     D in index order, so the last bit can differ from libtorch's
 *                                     blocked kernels -- the tests bound that difference
 *   2. scores *= scale                scale materialised in the storage type first
 *   3. mask                           causal: key j > query i gets -inf (tril(ones(Lq, Lk)), lines
 *                                     103-116); bool mask: false gets -inf; additive mask: added in
 *                                     double and rounded (mask_kind 0 none, 1 bool bytes, 2 additive
 *                                     of the storage type; mask is [B, Hq, Lq, Lk] contiguous)
 *   4. softmax over keys              po_softmax_lastdim's arithmetic
 *   5. out = attn v                   float accumulation over keys in index order
 * Returns 0, or 1 for arguments the reference rejects. */
int po_sdpa(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t Hq, int64_t Hkv,
            int64_t Lq, int64_t Lk, int64_t D, double scale, int causal, const void* mask, int mask_kind,
            int dt) {
    if (Hkv <= 0 || Hq % Hkv) return 1;
    if (causal && mask_kind) return 1;
    const int64_t rep = Hq / Hkv;
    const double scale_dt = rounded(scale, dt);
    const size_t es = elem_size(dt);
    int failed = 0;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t qo = ((b * Hq + h) * Lq) * D;
            const int64_t ko = ((b * Hkv + h / rep) * Lk) * D;
            void* row = malloc((size_t)(Lk > 0 ? Lk : 1) * es);      /* scores, then attn, of one query */
            if (!row) { failed = 1; continue; }
            for (int64_t i = 0; i < Lq; ++i) {
                for (int64_t j = 0; j < Lk; ++j) {
                    float acc = 0.f;
                    for (int64_t d = 0; d < D; ++d)
                        acc += (float)load(q, qo + i * D + d, dt) * (float)load(k, ko + j * D + d, dt);
                    double s = rounded((double)acc, dt);             /* bmm output */
                    s = rounded(s * scale_dt, dt);                   /* mul by scalar */
                    if (causal) {
                        if (j > i) s = -INFINITY;
                    } else if (mask_kind == 1) {
                        if (!((const uint8_t*)mask)[((b * Hq + h) * Lq + i) * Lk + j]) s = -INFINITY;
                    } else if (mask_kind == 2) {
                        s = rounded(s + load(mask, ((b * Hq + h) * Lq + i) * Lk + j, dt), dt);
                    }
                    store(row, j, dt, s);
                }
                softmax_row(row, row, 0, Lk, dt);
                for (int64_t d = 0; d < D; ++d) {
                    float acc = 0.f;
                    for (int64_t j = 0; j < Lk; ++j)
                        acc += (float)load(row, j, dt) * (float)load(v, ko + j * D + d, dt);
                    store(out, qo + i * D + d, dt, (double)acc);
                }
            }
            free(row);
        }
    return failed ? 2 : 0;
}
