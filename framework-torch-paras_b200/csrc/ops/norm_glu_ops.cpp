// RMSNorm, SwiGLU and rotate_half operators of the `paras` device, each one launch of a
// hand-written kernel through the C ABI.
//
// Operator surface kept from the reference:
//   aten::rms_norm(input, normalized_shape, weight?, eps?)       csrc/ops/rms_swiglu_ops.cpp:43-75,90-92
//   torch_paras::swiglu(x, gate) = x * silu(gate)  (PrivateUse1 + CPU)   rms_swiglu_ops.cpp:83-110
//   paras::rms_norm(input, weight, eps) -> (out, rstd)           csrc/ops/fused_ops.cpp:43-88
//   paras::rms_norm_backward                                      fused_ops.cpp:90-157
//   paras::swiglu(gate, up) / swiglu_backward                     fused_ops.cpp:162-229
//   paras::rotate_half / rotate_half_backward                     fused_ops.cpp:234-302
// Note the argument order: torch_paras::swiglu gates its SECOND argument, paras::swiglu its
// first.  The composite entry points (aten::rms_norm, torch_paras::swiglu) round to the
// tensor dtype after every step in the reference; the kernels reproduce that
// (PARAS_ROUND_PER_OP) so 16-bit results agree.
#include <torch/library.h>
#include <torch/csrc/autograd/custom_function.h>

#include "core/device_runtime.h"

namespace paras {
namespace {

using at::Tensor;

int checked_dtype(const Tensor& t, const char* what) {
    const int dt = dtype_code(t.scalar_type());
    TORCH_CHECK(dt >= 0, "paras ", what, ": unsupported dtype ", t.scalar_type(),
                " (float32, bfloat16 and float16 are supported)");
    return dt;
}

Tensor rms_norm_aten(const Tensor& input, at::IntArrayRef normalized_shape,
                     const std::optional<Tensor>& weight, std::optional<double> eps) {
    PARAS_TRACE_OP("rms_norm");
    const int64_t nd = int64_t(normalized_shape.size());
    TORCH_CHECK(nd >= 1, "paras rms_norm: normalized_shape must be non-empty");
    TORCH_CHECK(input.dim() >= nd, "paras rms_norm: input has fewer dims than normalized_shape");
    int64_t H = 1;
    for (int64_t i = 0; i < nd; ++i) {
        TORCH_CHECK(input.size(input.dim() - nd + i) == normalized_shape[i],
                    "paras rms_norm: normalized_shape does not match the trailing dims of input");
        H *= normalized_shape[i];
    }
    const bool has_w = weight.has_value() && weight->defined();
    if (has_w)
        TORCH_CHECK(weight->sizes().equals(normalized_shape),
                    "paras rms_norm: weight shape must equal normalized_shape");
    const int dt = checked_dtype(input, "rms_norm");
    if (has_w)
        TORCH_CHECK(weight->scalar_type() == input.scalar_type(),
                    "paras rms_norm: weight dtype must equal input dtype");
    const int gpu = Runtime::get().gpu_of(input);
    c10::DeviceGuard guard(input.device());
    Tensor x = input.contiguous();
    Tensor w = has_w ? weight->contiguous() : Tensor();
    Tensor out = at::empty_like(x);
    const int64_t rows = H > 0 ? x.numel() / H : 0;
    PARAS_ABI(paras_b200_rmsnorm_fwd(gpu, x.data_ptr(), has_w ? w.data_ptr() : nullptr,
                                     out.data_ptr(), nullptr, rows, H, eps.value_or(1e-6), dt,
                                     PARAS_ROUND_PER_OP, nullptr));
    return out;
}

std::tuple<Tensor, Tensor> rms_norm_fused(const Tensor& input, const Tensor& weight, double eps) {
    PARAS_TRACE_OP("paras::rms_norm");
    TORCH_CHECK(input.dim() >= 1, "paras rms_norm: input must have rank >= 1");
    const int dt = checked_dtype(input, "rms_norm");
    const int gpu = Runtime::get().gpu_of(input);
    c10::DeviceGuard guard(input.device());
    Tensor x = input.contiguous();
    Tensor w = weight.contiguous();
    const int64_t H = x.size(-1);
    const int64_t rows = H > 0 ? x.numel() / H : 0;
    TORCH_CHECK(w.numel() == H, "paras rms_norm: weight size must match the last dimension");
    TORCH_CHECK(w.scalar_type() == x.scalar_type(), "paras rms_norm: weight dtype must equal input dtype");
    Tensor out = at::empty_like(x);
    Tensor rstd = at::empty({rows}, x.options().dtype(c10::kFloat));
    PARAS_ABI(paras_b200_rmsnorm_fwd(gpu, x.data_ptr(), w.data_ptr(), out.data_ptr(),
                                     rows ? rstd.data_ptr<float>() : nullptr, rows, H, eps, dt,
                                     PARAS_ROUND_ONCE, nullptr));
    return {out, rstd};
}

std::tuple<Tensor, Tensor> rms_norm_backward(const Tensor& grad_out, const Tensor& input,
                                             const Tensor& weight, const Tensor& rstd) {
    PARAS_TRACE_OP("paras::rms_norm_backward");
    const int dt = checked_dtype(input, "rms_norm_backward");
    const int gpu = Runtime::get().gpu_of(input);
    c10::DeviceGuard guard(input.device());
    Tensor go = grad_out.contiguous(), x = input.contiguous(), w = weight.contiguous();
    Tensor r = rstd.contiguous();
    const int64_t H = x.size(-1);
    const int64_t rows = H > 0 ? x.numel() / H : 0;
    TORCH_CHECK(go.numel() == x.numel() && w.numel() == H && r.numel() == rows,
                "paras rms_norm_backward: shape mismatch");
    TORCH_CHECK(go.scalar_type() == x.scalar_type() && w.scalar_type() == x.scalar_type() &&
                    r.scalar_type() == c10::kFloat,
                "paras rms_norm_backward: dtype mismatch");
    Tensor gx = at::empty_like(x);
    Tensor gw = at::empty({H}, w.options());
    PARAS_ABI(paras_b200_rmsnorm_bwd(gpu, go.data_ptr(), x.data_ptr(), w.data_ptr(),
                                     rows ? r.data_ptr<float>() : nullptr, gx.data_ptr(),
                                     gw.data_ptr(), rows, H, dt, nullptr));
    return {gx, gw};
}

Tensor swiglu_fused(const Tensor& gate, const Tensor& up) {
    PARAS_TRACE_OP("paras::swiglu");
    TORCH_CHECK(gate.sizes() == up.sizes(), "paras swiglu: gate and up must have the same shape");
    TORCH_CHECK(gate.scalar_type() == up.scalar_type(), "paras swiglu: gate and up must have the same dtype");
    const int dt = checked_dtype(gate, "swiglu");
    const int gpu = Runtime::get().gpu_of(gate);
    c10::DeviceGuard guard(gate.device());
    Tensor g = gate.contiguous(), u = up.contiguous();
    Tensor out = at::empty_like(g);
    PARAS_ABI(paras_b200_swiglu_fwd(gpu, g.data_ptr(), u.data_ptr(), out.data_ptr(), out.numel(), dt,
                                    PARAS_ROUND_ONCE, nullptr));
    return out;
}

std::tuple<Tensor, Tensor> swiglu_backward(const Tensor& grad_out, const Tensor& gate,
                                           const Tensor& up) {
    PARAS_TRACE_OP("paras::swiglu_backward");
    TORCH_CHECK(gate.sizes() == up.sizes() && grad_out.sizes() == gate.sizes(),
                "paras swiglu_backward: shape mismatch");
    TORCH_CHECK(gate.scalar_type() == up.scalar_type() && grad_out.scalar_type() == gate.scalar_type(),
                "paras swiglu_backward: dtype mismatch");
    const int dt = checked_dtype(gate, "swiglu_backward");
    const int gpu = Runtime::get().gpu_of(gate);
    c10::DeviceGuard guard(gate.device());
    Tensor go = grad_out.contiguous(), g = gate.contiguous(), u = up.contiguous();
    Tensor gg = at::empty_like(g), gu = at::empty_like(u);
    PARAS_ABI(paras_b200_swiglu_bwd(gpu, go.data_ptr(), g.data_ptr(), u.data_ptr(), gg.data_ptr(),
                                    gu.data_ptr(), g.numel(), dt, nullptr));
    return {gg, gu};
}

// torch_paras::swiglu(x, gate): broadcasting allowed, silu(gate) rounded before the multiply.
Tensor swiglu_composite(const Tensor& x, const Tensor& gate) {
    PARAS_TRACE_OP("swiglu");
    if (x.device().type() != kDevice) return x * at::silu(gate);  // CPU registration
    TORCH_CHECK(x.scalar_type() == gate.scalar_type(), "paras swiglu: x and gate must have the same dtype");
    const int dt = checked_dtype(x, "swiglu");
    const int gpu = Runtime::get().gpu_of(x);
    c10::DeviceGuard guard(x.device());
    auto bc = at::broadcast_tensors({x, gate});
    Tensor xb = bc[0].contiguous(), gb = bc[1].contiguous();
    Tensor out = at::empty_like(xb);
    PARAS_ABI(paras_b200_swiglu_fwd(gpu, gb.data_ptr(), xb.data_ptr(), out.data_ptr(), out.numel(), dt,
                                    PARAS_ROUND_PER_OP, nullptr));
    return out;
}

Tensor rotate_half_impl(const Tensor& x, int backward, const char* name) {
    TORCH_CHECK(x.dim() >= 1, "paras ", name, ": input must have rank >= 1");
    const int64_t D = x.size(-1);
    TORCH_CHECK(D % 2 == 0, "paras ", name, ": last dimension must be even");
    const int dt = checked_dtype(x, name);
    const int gpu = Runtime::get().gpu_of(x);
    c10::DeviceGuard guard(x.device());
    Tensor xc = x.contiguous();
    Tensor out = at::empty_like(xc);
    const int64_t rows = D > 0 ? xc.numel() / D : 0;
    PARAS_ABI(paras_b200_rotate_half(gpu, xc.data_ptr(), out.data_ptr(), rows, D, dt, backward, nullptr));
    return out;
}

Tensor rotate_half(const Tensor& x) {
    PARAS_TRACE_OP("paras::rotate_half");
    return rotate_half_impl(x, 0, "rotate_half");
}

Tensor rotate_half_backward(const Tensor& grad_out) {
    PARAS_TRACE_OP("paras::rotate_half_backward");
    return rotate_half_impl(grad_out, 1, "rotate_half_backward");
}

// ---- autograd for F.rms_norm on `paras` tensors -------------------------------------------
// The reference's aten::rms_norm is a composition of at:: operators that autograd follows
// (rms_swiglu_ops.cpp:66-73).  With a fused backend kernel in its place the gradient is tied on
// here: inputs that require grad go through paras::rms_norm + paras::rms_norm_backward
// (fused_ops.cpp:43-157), over the trailing normalized_shape dims flattened into one.
struct RmsNormFunction : public torch::autograd::Function<RmsNormFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& x2d, const Tensor& w, double eps) {
        auto [out, rstd] = rms_norm_fused(x2d, w, eps);
        ctx->save_for_backward({x2d, w, rstd});
        return out;
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grads) {
        const auto saved = ctx->get_saved_variables();
        auto [gx, gw] = rms_norm_backward(grads[0], saved[0], saved[1], saved[2]);
        return {gx, gw, Tensor()};
    }
};

Tensor rms_norm_autograd(const Tensor& input, at::IntArrayRef normalized_shape,
                         const std::optional<Tensor>& weight, std::optional<double> eps) {
    const bool has_w = weight.has_value() && weight->defined();
    const bool needs_grad = at::GradMode::is_enabled() &&
                            (input.requires_grad() || (has_w && weight->requires_grad()));
    if (!needs_grad) {
        at::AutoDispatchBelowADInplaceOrView below;
        return at::rms_norm(input, normalized_shape, weight, eps);
    }
    const int64_t nd = int64_t(normalized_shape.size());
    TORCH_CHECK(nd >= 1 && input.dim() >= nd, "paras rms_norm: normalized_shape does not fit the input");
    int64_t H = 1;
    for (int64_t i = 0; i < nd; ++i) {
        TORCH_CHECK(input.size(input.dim() - nd + i) == normalized_shape[i],
                    "paras rms_norm: normalized_shape does not match the trailing dims of input");
        H *= normalized_shape[i];
    }
    if (has_w)
        TORCH_CHECK(weight->sizes().equals(normalized_shape),
                    "paras rms_norm: weight shape must equal normalized_shape");
    Tensor w = has_w ? weight->reshape({H}) : at::ones({H}, input.options());
    Tensor out = RmsNormFunction::apply(input.reshape({-1, H}), w, eps.value_or(1e-6));
    return out.reshape(input.sizes());
}

}  // namespace
}  // namespace paras

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) { m.impl("aten::rms_norm", &paras::rms_norm_aten); }
TORCH_LIBRARY_IMPL(aten, AutogradPrivateUse1, m) { m.impl("aten::rms_norm", &paras::rms_norm_autograd); }

TORCH_LIBRARY_FRAGMENT(torch_paras, m) { m.def("swiglu(Tensor x, Tensor gate) -> Tensor"); }
TORCH_LIBRARY_IMPL(torch_paras, PrivateUse1, m) { m.impl("swiglu", &paras::swiglu_composite); }
TORCH_LIBRARY_IMPL(torch_paras, CPU, m) { m.impl("swiglu", &paras::swiglu_composite); }

TORCH_LIBRARY(paras, m) {
    m.def("rms_norm(Tensor input, Tensor weight, float eps) -> (Tensor, Tensor)");
    m.def("rms_norm_backward(Tensor grad_out, Tensor input, Tensor weight, Tensor rstd) -> (Tensor, Tensor)");
    m.def("swiglu(Tensor gate, Tensor up) -> Tensor");
    m.def("swiglu_backward(Tensor grad_out, Tensor gate, Tensor up) -> (Tensor, Tensor)");
    m.def("rotate_half(Tensor x) -> Tensor");
    m.def("rotate_half_backward(Tensor grad_out) -> Tensor");
}

TORCH_LIBRARY_IMPL(paras, PrivateUse1, m) {
    m.impl("rms_norm", &paras::rms_norm_fused);
    m.impl("rms_norm_backward", &paras::rms_norm_backward);
    m.impl("swiglu", &paras::swiglu_fused);
    m.impl("swiglu_backward", &paras::swiglu_backward);
    m.impl("rotate_half", &paras::rotate_half);
    m.impl("rotate_half_backward", &paras::rotate_half_backward);
}
