// Matrix products of the `paras` device: the projections on either side of the attention /
// RMSNorm / SwiGLU path.
//
// Operator surface kept from the reference (csrc/ops/vision_ops.cpp):
//   aten::mm, aten::bmm, aten::addmm          mm_out / bmm_out / addmm_out, 388-423
//   aten::linear                              LinearFunction::forward, 248-309
// There every product copies both operands to the host, runs libtorch's CPU GEMM and copies the
// result back.  Here 16-bit operands with 16-byte aligned rows go to the tcgen05 kernel behind
// paras_b200_gemm; anything else (fp32 -- a TF32 product would not meet the 1e-4 tolerance the
// reference's tests use --, odd leading dimensions, general alpha/beta) keeps the reference's
// host route, so results there are the reference's own.
//
// New, without a counterpart in the reference:
//   paras::swiglu_linear(x, w_gate, w_up) = paras::swiglu(linear(x, w_gate), linear(x, w_up))
// as one kernel: the gate and up projections share one pass over x and SwiGLU runs in the
// GEMM's epilogue, so the two [rows, F] intermediates never reach memory.
#include <torch/library.h>

#include "core/device_runtime.h"

namespace paras {
namespace {

using at::Tensor;

bool sixteen_bit(const Tensor& t) {
    return t.scalar_type() == c10::kBFloat16 || t.scalar_type() == c10::kHalf;
}

// A [.., rows, cols] view whose rows are contiguous and 16-byte aligned, copying if needed.
Tensor row_major(const Tensor& t) {
    const int64_t ld = t.stride(-2);
    const bool ok = t.stride(-1) == 1 && ld % 8 == 0 && ld >= t.size(-1) &&
                    (t.dim() < 3 || t.stride(0) % 8 == 0) &&
                    reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
    return ok ? t : t.contiguous();
}

struct Operand {
    Tensor t;      // keeps the memory alive
    int layout;    // PARAS_GEMM_B_NK or PARAS_GEMM_B_KN
    int64_t ld, batch_stride;
};

// mat2 as the kernel's B operand: [.., K, N] with rows of N, or -- when it is the transposed
// view of a row-major [N, K] matrix, as in x @ w.t() -- that matrix itself.
Operand as_b(const Tensor& mat2) {
    const int d = int(mat2.dim());
    const bool aligned = reinterpret_cast<uintptr_t>(mat2.data_ptr()) % 16 == 0 &&
                         (d < 3 || mat2.stride(0) % 8 == 0);
    if (aligned && mat2.stride(-2) == 1 && mat2.stride(-1) % 8 == 0 && mat2.stride(-1) >= mat2.size(-2))
        return {mat2, PARAS_GEMM_B_NK, mat2.stride(-1), d == 3 ? mat2.stride(0) : 0};
    Tensor b = row_major(mat2);
    return {b, PARAS_GEMM_B_KN, b.stride(-2), d == 3 ? b.stride(0) : 0};
}

// Runs the kernel; false when the library says the operands are not for it.
bool try_gemm(const Tensor& a, const Operand& b, const Tensor* up_weight, const Tensor* bias,
              Tensor& out, int64_t batch, int64_t M, int64_t N, int64_t K) {
    paras_gemm_args g{};
    g.a = a.data_ptr();
    g.b = b.t.data_ptr();
    g.b2 = up_weight ? up_weight->data_ptr() : nullptr;
    g.bias = bias ? bias->data_ptr() : nullptr;
    g.c = out.data_ptr();
    g.M = M; g.N = N; g.K = K;
    g.lda = a.stride(-2); g.ldb = b.ld; g.ldc = out.stride(-2);
    g.batch = batch;
    g.stride_a = a.dim() == 3 ? a.stride(0) : 0;
    g.stride_b = b.batch_stride;
    g.stride_c = out.dim() == 3 ? out.stride(0) : 0;
    g.dtype = dtype_code(a.scalar_type());
    g.b_layout = b.layout;
    g.epilogue = up_weight ? PARAS_GEMM_EPI_SWIGLU : (bias ? PARAS_GEMM_EPI_BIAS : PARAS_GEMM_EPI_NONE);
    g.gpu = Runtime::get().gpu_of(a);
    g.stream = nullptr;
    const int st = paras_b200_gemm(&g);
    if (st == PARAS_E_UNSUPPORTED) return false;
    TORCH_CHECK(st == PARAS_OK, paras_b200_last_error());
    return true;
}

Tensor host(const Tensor& t) { return t.to(c10::kCPU); }

Tensor mm(const Tensor& self, const Tensor& mat2) {
    PARAS_TRACE_OP("mm");
    TORCH_CHECK(self.dim() == 2 && mat2.dim() == 2, "paras mm: both arguments must be matrices");
    TORCH_CHECK(self.size(1) == mat2.size(0), "paras mm: shapes cannot be multiplied (", self.size(0),
                "x", self.size(1), " and ", mat2.size(0), "x", mat2.size(1), ")");
    TORCH_CHECK(self.scalar_type() == mat2.scalar_type(), "paras mm: operands must have the same dtype");
    c10::DeviceGuard guard(self.device());
    if (sixteen_bit(self) && self.size(1) > 0) {
        Tensor a = row_major(self);
        Operand b = as_b(mat2);
        Tensor out = at::empty({self.size(0), mat2.size(1)}, self.options());
        if (try_gemm(a, b, nullptr, nullptr, out, 1, self.size(0), mat2.size(1), self.size(1))) return out;
    }
    return at::mm(host(self), host(mat2)).to(self.device());
}

Tensor bmm(const Tensor& self, const Tensor& mat2) {
    PARAS_TRACE_OP("bmm");
    TORCH_CHECK(self.dim() == 3 && mat2.dim() == 3, "paras bmm: both arguments must be 3-D");
    TORCH_CHECK(self.size(0) == mat2.size(0) && self.size(2) == mat2.size(1),
                "paras bmm: shapes cannot be multiplied");
    TORCH_CHECK(self.scalar_type() == mat2.scalar_type(), "paras bmm: operands must have the same dtype");
    c10::DeviceGuard guard(self.device());
    if (sixteen_bit(self) && self.size(2) > 0) {
        Tensor a = row_major(self);
        Operand b = as_b(mat2);
        Tensor out = at::empty({self.size(0), self.size(1), mat2.size(2)}, self.options());
        if (try_gemm(a, b, nullptr, nullptr, out, self.size(0), self.size(1), mat2.size(2), self.size(2)))
            return out;
    }
    return at::bmm(host(self), host(mat2)).to(self.device());
}

Tensor addmm(const Tensor& self, const Tensor& mat1, const Tensor& mat2, const at::Scalar& beta,
             const at::Scalar& alpha) {
    PARAS_TRACE_OP("addmm");
    TORCH_CHECK(mat1.dim() == 2 && mat2.dim() == 2 && mat1.size(1) == mat2.size(0),
                "paras addmm: shapes cannot be multiplied");
    c10::DeviceGuard guard(mat1.device());
    const int64_t N = mat2.size(1);
    const bool bias_like = (self.dim() == 1 && self.size(0) == N) ||
                           (self.dim() == 2 && self.size(0) == 1 && self.size(1) == N);
    if (sixteen_bit(mat1) && mat2.scalar_type() == mat1.scalar_type() &&
        self.scalar_type() == mat1.scalar_type() && bias_like && mat1.size(1) > 0 &&
        beta.toDouble() == 1.0 && alpha.toDouble() == 1.0) {
        Tensor a = row_major(mat1);
        Operand b = as_b(mat2);
        Tensor bias = self.reshape({N}).contiguous();
        Tensor out = at::empty({mat1.size(0), N}, mat1.options());
        if (try_gemm(a, b, nullptr, &bias, out, 1, mat1.size(0), N, mat1.size(1))) return out;
    }
    return at::addmm(host(self), host(mat1), host(mat2), beta, alpha).to(mat1.device());
}

Tensor linear(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias) {
    PARAS_TRACE_OP("linear");
    TORCH_CHECK(weight.dim() == 2, "paras linear: weight must be [out_features, in_features]");
    TORCH_CHECK(input.dim() >= 1 && input.size(-1) == weight.size(1),
                "paras linear: input's last dimension must equal in_features");
    const bool has_bias = bias.has_value() && bias->defined() && bias->numel() > 0;
    c10::DeviceGuard guard(input.device());
    const int64_t K = weight.size(1), N = weight.size(0);
    if (sixteen_bit(input) && weight.scalar_type() == input.scalar_type() && K > 0 &&
        (!has_bias || (bias->scalar_type() == input.scalar_type() && bias->numel() == N))) {
        Tensor x = row_major(input.reshape({-1, K}));
        Tensor w = row_major(weight);
        Tensor b = has_bias ? bias->contiguous() : Tensor();
        Tensor out = at::empty({x.size(0), N}, input.options());
        Operand wb{w, PARAS_GEMM_B_NK, w.stride(0), 0};
        if (try_gemm(x, wb, nullptr, has_bias ? &b : nullptr, out, 1, x.size(0), N, K)) {
            auto shape = input.sizes().vec();
            shape.back() = N;
            return out.reshape(shape);
        }
    }
    return at::linear(host(input), host(weight), has_bias ? host(*bias) : Tensor()).to(input.device());
}

Tensor swiglu_linear(const Tensor& x, const Tensor& w_gate, const Tensor& w_up) {
    PARAS_TRACE_OP("paras::swiglu_linear");
    TORCH_CHECK(w_gate.dim() == 2 && w_up.sizes() == w_gate.sizes(),
                "paras swiglu_linear: the two weights must be [features, in_features] of equal shape");
    TORCH_CHECK(x.dim() >= 1 && x.size(-1) == w_gate.size(1),
                "paras swiglu_linear: input's last dimension must equal in_features");
    TORCH_CHECK(sixteen_bit(x) && w_gate.scalar_type() == x.scalar_type() &&
                    w_up.scalar_type() == x.scalar_type(),
                "paras swiglu_linear: bfloat16 or float16 operands of one dtype");
    c10::DeviceGuard guard(x.device());
    const int64_t K = w_gate.size(1), F = w_gate.size(0);
    Tensor a = row_major(x.reshape({-1, K}));
    Tensor wg = row_major(w_gate), wu = row_major(w_up);
    if (wu.stride(0) != wg.stride(0)) { wg = wg.contiguous(); wu = wu.contiguous(); }
    Tensor out = at::empty({a.size(0), F}, x.options());
    Operand wb{wg, PARAS_GEMM_B_NK, wg.stride(0), 0};
    TORCH_CHECK(try_gemm(a, wb, &wu, nullptr, out, 1, a.size(0), F, K), paras_b200_last_error());
    auto shape = x.sizes().vec();
    shape.back() = F;
    return out.reshape(shape);
}

// ---- RMSNorm folded into the projection that follows it ------------------------------------
// linear(rms_norm(x, w_norm), W) = rstd[row] * (x @ (W o w_norm)^T): the per-column norm weight moves
// into the projection weight (once per weight, fold_norm_weight), the per-row rstd into the GEMM's
// epilogue.  What the reference runs as rms_norm (csrc/ops/rms_swiglu_ops.cpp:43-75, fused_ops.cpp:
// 43-88) followed by linear (vision_ops.cpp:248-309) -- a write and a read of the normalised
// activations in between -- becomes one read of x for rstd and the GEMM.  New operators, 16-bit.
Tensor fold_norm_weight(const Tensor& weight, const Tensor& norm_weight) {
    PARAS_TRACE_OP("paras::fold_norm_weight");
    TORCH_CHECK(weight.dim() == 2 && norm_weight.dim() == 1 && norm_weight.size(0) == weight.size(1),
                "paras fold_norm_weight: weight [out_features, in_features], norm_weight [in_features]");
    TORCH_CHECK(dtype_code(weight.scalar_type()) >= 0 && norm_weight.scalar_type() == weight.scalar_type(),
                "paras fold_norm_weight: float32, bfloat16 or float16 tensors of one dtype");
    c10::DeviceGuard guard(weight.device());
    Tensor w = weight.contiguous(), nw = norm_weight.contiguous();
    Tensor out = at::empty_like(w);
    PARAS_ABI(paras_b200_scale_columns(Runtime::get().gpu_of(w), w.data_ptr(), nw.data_ptr(), out.data_ptr(),
                                       w.size(0), w.size(1), dtype_code(w.scalar_type()), nullptr));
    return out;
}

Tensor rms_norm_linear_folded(const Tensor& x, const Tensor& folded_weight, double eps) {
    PARAS_TRACE_OP("paras::rms_norm_linear_folded");
    TORCH_CHECK(folded_weight.dim() == 2 && x.dim() >= 1 && x.size(-1) == folded_weight.size(1),
                "paras rms_norm_linear: input's last dimension must equal in_features");
    TORCH_CHECK(sixteen_bit(x) && folded_weight.scalar_type() == x.scalar_type(),
                "paras rms_norm_linear: bfloat16 or float16 operands of one dtype");
    c10::DeviceGuard guard(x.device());
    const int64_t K = folded_weight.size(1), N = folded_weight.size(0);
    Tensor a = x.reshape({-1, K}).contiguous();
    Tensor w = row_major(folded_weight);
    const int gpu = Runtime::get().gpu_of(a);
    Tensor rstd = at::empty({a.size(0)}, a.options().dtype(c10::kFloat));
    Tensor out = at::empty({a.size(0), N}, x.options());
    if (a.size(0) > 0) {
        PARAS_ABI(paras_b200_rms_rstd(gpu, a.data_ptr(), rstd.data_ptr<float>(), a.size(0), K, eps,
                                      dtype_code(a.scalar_type()), nullptr));
        paras_gemm_args g{};
        g.a = a.data_ptr(); g.b = w.data_ptr(); g.c = out.data_ptr();
        g.M = a.size(0); g.N = N; g.K = K;
        g.lda = a.stride(0); g.ldb = w.stride(0); g.ldc = out.stride(0);
        g.batch = 1;
        g.dtype = dtype_code(a.scalar_type());
        g.b_layout = PARAS_GEMM_B_NK;
        g.epilogue = PARAS_GEMM_EPI_ROWSCALE;
        g.row_scale = rstd.data_ptr<float>();
        g.gpu = gpu;
        PARAS_ABI(paras_b200_gemm(&g));
    }
    auto shape = x.sizes().vec();
    shape.back() = N;
    return out.reshape(shape);
}

Tensor rms_norm_linear(const Tensor& x, const Tensor& norm_weight, const Tensor& weight, double eps) {
    PARAS_TRACE_OP("paras::rms_norm_linear");
    return rms_norm_linear_folded(x, fold_norm_weight(weight, norm_weight), eps);
}

// aten::linear with inputs that require grad: as a product autograd knows (matmul -> mm / bmm,
// whose derivative formulas call mm on this device again), like the reference's own
// differentiable linear (vision_ops.cpp:248-309).  Without grad the fused kernel runs.
Tensor linear_autograd(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias) {
    const bool has_bias = bias.has_value() && bias->defined();
    const bool needs_grad = at::GradMode::is_enabled() &&
                            (input.requires_grad() || weight.requires_grad() || (has_bias && bias->requires_grad()));
    if (!needs_grad) {
        at::AutoDispatchBelowADInplaceOrView below;
        return at::linear(input, weight, bias);
    }
    TORCH_CHECK(weight.dim() == 2, "paras linear: weight must be [out_features, in_features]");
    Tensor x2d = input.reshape({-1, input.size(-1)});
    Tensor out = has_bias ? at::addmm(*bias, x2d, weight.t()) : at::mm(x2d, weight.t());
    auto shape = input.sizes().vec();
    shape.back() = weight.size(0);
    return out.reshape(shape);
}

}  // namespace
}  // namespace paras

TORCH_LIBRARY_IMPL(aten, AutogradPrivateUse1, m) { m.impl("aten::linear", &paras::linear_autograd); }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("aten::mm", &paras::mm);
    m.impl("aten::bmm", &paras::bmm);
    m.impl("aten::addmm", &paras::addmm);
    m.impl("aten::linear", &paras::linear);
}

TORCH_LIBRARY_FRAGMENT(paras, m) {
    m.def("swiglu_linear(Tensor x, Tensor w_gate, Tensor w_up) -> Tensor");
    m.def("fold_norm_weight(Tensor weight, Tensor norm_weight) -> Tensor");
    m.def("rms_norm_linear(Tensor x, Tensor norm_weight, Tensor weight, float eps) -> Tensor");
    m.def("rms_norm_linear_folded(Tensor x, Tensor folded_weight, float eps) -> Tensor");
}
TORCH_LIBRARY_IMPL(paras, PrivateUse1, m) {
    m.impl("swiglu_linear", &paras::swiglu_linear);
    m.impl("fold_norm_weight", &paras::fold_norm_weight);
    m.impl("rms_norm_linear", &paras::rms_norm_linear);
    m.impl("rms_norm_linear_folded", &paras::rms_norm_linear_folded);
}
