// scaled_dot_product_attention on `paras:N`: one fused flash-attention launch through the
// C ABI instead of the reference's composition.
//
// Reference being replaced: sdpa_math, csrc/ops/attention_ops.cpp:71-136, registered as
// aten::_scaled_dot_product_attention_math (140-142) -- repeat_interleave + matmul + mul +
// ones/tril/logical_not/masked_fill + softmax + matmul, each a full pass over a
// [B,H,Lq,Lk] score tensor.  Same argument checks and error behaviour (RuntimeError):
// rank >= 3, is_causal excludes attn_mask, query heads must be a multiple of kv heads with
// enable_gqa, default scale 1/sqrt(E), causal mask top-left aligned.
//
// Both the math op and the top-level aten::scaled_dot_product_attention are registered for
// PrivateUse1 (the reference suggests the second at attention_ops.cpp:144-150); the
// top-level registration keeps PyTorch from pre-converting a bool mask into an additive one.
// Dropout (the reference's Philox stream, or a caller's dropout_mask) and the attention weights
// that the math op returns need every normalised weight: those calls take a two-pass CUDA-core
// kernel instead of the flash kernels (attention_ops.cpp:128-135, random_ops.cpp:140-176).
#include <torch/library.h>
#include <torch/csrc/autograd/custom_function.h>

#include <cmath>
#include <cstdlib>

#include "core/device_runtime.h"

namespace paras {
namespace {

using at::Tensor;

// (..., H, L, E) -> [B, H, L, E] with a unit stride on E; 3-D inputs are (B, L, E) with one head.
Tensor as_bhle(const Tensor& t) {
    Tensor r = t;
    if (r.dim() == 3) r = r.unsqueeze(1);
    else if (r.dim() > 4) r = r.reshape({-1, r.size(-3), r.size(-2), r.size(-1)});
    if (r.size(-1) > 1 && r.stride(-1) != 1) r = r.contiguous();
    return r;
}

bool ref_scale_rounding() {
    static const bool on = [] {
        const char* e = std::getenv("PARAS_SDPA_TRUE_SCALE");
        return !(e && std::atoi(e) != 0);
    }();
    return on;
}

// Largest attention-weights tensor the math op will materialise (elements): 2^28 = 512 MB in 16 bit.
constexpr int64_t kMaxWeightsElements = int64_t(1) << 28;

// The Philox (seed, sequence) pair of one dropout draw.
using RngState = std::pair<uint64_t, uint64_t>;

// What a general gradient call adds to the forward's arguments: the output's gradient in, the three
// gradients out, and the dropout draw of the forward it differentiates.
struct GradRequest {
    const Tensor* grad_out;
    const RngState* rng;
    Tensor dq, dk, dv;
};

// Validates and lays out one attention call.  Without `grad` it runs the forward (drawing dropout
// counters when it needs them; `rng_used` receives them); with `grad` it runs the general backward of
// exactly that call instead and returns an undefined tensor.
Tensor sdpa_forward(const Tensor& query, const Tensor& key, const Tensor& value,
                    const std::optional<Tensor>& attn_mask, double dropout_p, bool is_causal,
                    std::optional<double> scale, bool enable_gqa,
                    const std::optional<Tensor>& dropout_mask = std::nullopt, Tensor* weights = nullptr,
                    RngState* rng_used = nullptr, GradRequest* grad = nullptr) {
    TORCH_CHECK(query.dim() >= 3 && key.dim() >= 3 && value.dim() >= 3,
                "paras sdpa: query/key/value must be at least 3-D (..., seq, head_dim)");
    const bool has_mask = attn_mask.has_value() && attn_mask->defined();
    TORCH_CHECK(!(is_causal && has_mask),
                "paras sdpa: is_causal and attn_mask are mutually exclusive");
    TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "paras sdpa: dropout_p must be in [0, 1), got ", dropout_p);
    TORCH_CHECK(query.scalar_type() == key.scalar_type() && query.scalar_type() == value.scalar_type(),
                "paras sdpa: query, key and value must have the same dtype");
    const int dt = dtype_code(query.scalar_type());
    TORCH_CHECK(dt >= 0, "paras sdpa: unsupported dtype ", query.scalar_type(),
                " (float32, bfloat16 and float16 are supported)");
    TORCH_CHECK(key.device() == query.device() && value.device() == query.device(),
                "paras sdpa: query, key and value must be on the same device");
    Runtime& rt = Runtime::get();
    const int gpu = rt.gpu_of(query);

    Tensor q = as_bhle(query), k = as_bhle(key), v = as_bhle(value);
    const int64_t B = q.size(0), Hq = q.size(1), Lq = q.size(2), E = q.size(3);
    const int64_t Hkv = k.size(1), Lk = k.size(2);
    TORCH_CHECK(k.size(0) == B && v.size(0) == B, "paras sdpa: batch dimensions of query, key and value differ");
    TORCH_CHECK(k.size(3) == E, "paras sdpa: query and key head_dim differ");
    TORCH_CHECK(v.size(1) == Hkv && v.size(2) == Lk, "paras sdpa: key and value shapes differ");
    TORCH_CHECK(v.size(3) == E, "paras sdpa: value head_dim (", v.size(3), ") must equal query head_dim (", E,
                "): the kernels share one head dim; pad the narrower operand with zero columns");
    if (Hkv != Hq) {
        TORCH_CHECK(enable_gqa, "paras sdpa: key/value have ", Hkv, " heads but query has ", Hq,
                    "; pass enable_gqa=True for grouped-query attention");
        TORCH_CHECK(Hkv > 0 && Hq % Hkv == 0,
                    "paras sdpa: query heads must be a multiple of key/value heads for enable_gqa");
    }
    c10::DeviceGuard guard(query.device());
    Tensor out = grad ? Tensor() : at::empty({B, Hq, Lq, E}, q.options());

    paras_sdpa_args a{};
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.out = grad ? nullptr : out.data_ptr();
    a.dtype = dt;
    a.B = int32_t(B); a.Hq = int32_t(Hq); a.Hkv = int32_t(Hkv);
    a.Lq = int32_t(Lq); a.Lk = int32_t(Lk); a.D = int32_t(E);
    for (int i = 0; i < 3; ++i) {
        a.q_strides[i] = q.stride(i);
        a.k_strides[i] = k.stride(i);
        a.v_strides[i] = v.stride(i);
        a.o_strides[i] = grad ? 0 : out.stride(i);
    }
    Tensor mask;  // keeps a converted mask alive until the launch is queued
    if (has_mask) {
        mask = *attn_mask;
        TORCH_CHECK(mask.device() == query.device(), "paras sdpa: attn_mask must be on the query's device");
        if (mask.scalar_type() == c10::kBool) a.mask_kind = 1;
        else if (mask.scalar_type() == query.scalar_type()) a.mask_kind = 2;
        else if (mask.scalar_type() == c10::kFloat) a.mask_kind = 3;
        else { mask = mask.to(query.scalar_type()); a.mask_kind = 2; }
        // The reference adds the mask to scores of shape (..., Lq, Lk) (attention_ops.cpp:117-126), so
        // it broadcasts from the right against the query's own leading dims; only then does the mask
        // follow the query into [B, H, Lq, Lk] (a 3-D query's [B, Lq, Lk] mask is per batch element).
        std::vector<int64_t> score_shape(query.sizes().begin(), query.sizes().end() - 1);
        score_shape.push_back(Lk);
        TORCH_CHECK(mask.dim() <= int64_t(score_shape.size()),
                    "paras sdpa: attn_mask has more dimensions than the attention scores");
        mask = mask.expand(score_shape);
        if (query.dim() == 3) mask = mask.unsqueeze(1);
        else if (query.dim() > 4) mask = mask.reshape({-1, Hq, Lq, Lk});
        mask = mask.expand({B, Hq, Lq, Lk});
        a.mask = mask.data_ptr();
        for (int i = 0; i < 4; ++i) a.mask_strides[i] = mask.stride(i);
    }
    a.causal = is_causal ? 1 : 0;
    a.scale = scale.has_value() ? *scale : 1.0 / std::sqrt(double(E));
    a.flags = ref_scale_rounding() ? PARAS_SDPA_REF_SCALE : 0;
    a.gpu = gpu;
    a.stream = nullptr;
    Tensor dmask;   // keeps a converted dropout mask alive until the launch is queued
    if (dropout_p > 0.0 && Lk > 0 && B * Hq * Lq * E > 0) {
        a.dropout_p = dropout_p;
        if (dropout_mask.has_value() && dropout_mask->defined()) {
            dmask = *dropout_mask;
            TORCH_CHECK(dmask.device() == query.device(), "paras sdpa: dropout_mask must be on the query's device");
            if (dmask.scalar_type() == c10::kBool) a.dropout_mask_kind = 1;
            else if (dmask.scalar_type() == query.scalar_type()) a.dropout_mask_kind = 2;
            else if (dmask.scalar_type() == c10::kFloat) a.dropout_mask_kind = 3;
            else { dmask = dmask.to(query.scalar_type()); a.dropout_mask_kind = 2; }
            std::vector<int64_t> score_shape(query.sizes().begin(), query.sizes().end() - 1);
            score_shape.push_back(Lk);
            dmask = dmask.expand(score_shape);
            if (query.dim() == 3) dmask = dmask.unsqueeze(1);
            else if (query.dim() > 4) dmask = dmask.reshape({-1, Hq, Lq, Lk});
            dmask = dmask.expand({B, Hq, Lq, Lk});
            a.dropout_mask = dmask.data_ptr();
            for (int i = 0; i < 4; ++i) a.dropout_mask_strides[i] = dmask.stride(i);
        } else {
            // the counters the reference's native_dropout would draw for its [B,Hq,Lq,Lk] weights
            const RngState state = grad ? *grad->rng : rt.rng_draw(int(query.device().index()), B * Hq * Lq * Lk);
            a.rng_seed = state.first;
            a.rng_sequence = state.second;
            if (rng_used) *rng_used = state;
        }
    }
    if (grad) {
        TORCH_CHECK(grad->grad_out->sizes() == query.sizes(), "paras sdpa backward: the output's gradient has shape ",
                    grad->grad_out->sizes(), ", the output ", query.sizes());
        Tensor go = as_bhle(grad->grad_out->to(query.scalar_type()));
        Tensor dq = at::empty({B, Hq, Lq, E}, q.options()), dk = at::empty({B, Hkv, Lk, E}, q.options()),
               dv = at::empty({B, Hkv, Lk, E}, q.options());
        const int64_t gs[3] = {go.stride(0), go.stride(1), go.stride(2)};
        PARAS_ABI(paras_b200_sdpa_bwd_general(&a, go.data_ptr(), gs, dq.data_ptr(), dk.data_ptr(), dv.data_ptr()));
        grad->dq = dq.reshape(query.sizes());
        grad->dk = dk.reshape(key.sizes());
        grad->dv = dv.reshape(value.sizes());
        return Tensor();
    }
    if (weights) {
        TORCH_CHECK(B * Hq * Lq * Lk <= kMaxWeightsElements,
                    "paras sdpa: the attention weights [", B, ", ", Hq, ", ", Lq, ", ", Lk, "] are too large to "
                    "materialise; call F.scaled_dot_product_attention, which returns no weights and runs the "
                    "fused kernel");
        *weights = at::empty({B, Hq, Lq, Lk}, q.options());
        if (weights->numel() > 0 && Lk > 0) a.attn_out = weights->data_ptr();
    }
    PARAS_ABI(paras_b200_sdpa_fwd(&a));
    if (weights) {
        if (query.dim() == 3) *weights = weights->squeeze(1);
        else if (query.dim() > 4) {
            std::vector<int64_t> wshape(query.sizes().begin(), query.sizes().end() - 1);
            wshape.push_back(Lk);
            *weights = weights->reshape(wshape);
        }
    }

    if (query.dim() == 3) return out.squeeze(1);
    if (query.dim() > 4) {
        std::vector<int64_t> shape(query.sizes().begin(), query.sizes().end());
        return out.reshape(shape);
    }
    return out;
}

// aten::_scaled_dot_product_attention_math returns (output, attention weights after dropout) like the
// reference.  The weights are O(Lq * Lk) per head: this entry point therefore always runs the
// two-pass kernel, and refuses shapes whose weights exceed kMaxWeightsElements -- F.scaled_dot_product_
// attention (no weights) is the entry point for those.
std::tuple<Tensor, Tensor> sdpa_math(const Tensor& query, const Tensor& key, const Tensor& value,
                                     const std::optional<Tensor>& attn_mask, double dropout_p,
                                     bool is_causal, const std::optional<Tensor>& dropout_mask,
                                     std::optional<double> scale, bool enable_gqa) {
    PARAS_TRACE_OP("_scaled_dot_product_attention_math");
    Tensor weights;
    Tensor out = sdpa_forward(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa, dropout_mask,
                              &weights);
    return {out, weights};
}

Tensor sdpa(const Tensor& query, const Tensor& key, const Tensor& value,
            const std::optional<Tensor>& attn_mask, double dropout_p, bool is_causal,
            std::optional<double> scale, bool enable_gqa) {
    PARAS_TRACE_OP("scaled_dot_product_attention");
    return sdpa_forward(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa);
}


// ---- training: forward that also returns the row statistics, and the backward built on them ----
// paras::sdpa_train_forward(q, k, v, is_causal, scale) -> (out, lse);  paras::sdpa_backward(...)
// New operators (the reference differentiates through its composite); 4-D [B,H,L,E] 16-bit
// tensors, GQA by head count, no mask tensor.  Wrapped for autograd in torch_paras.nn.
std::tuple<Tensor, Tensor> sdpa_train_forward(const Tensor& query, const Tensor& key, const Tensor& value,
                                              bool is_causal, std::optional<double> scale) {
    PARAS_TRACE_OP("paras::sdpa_train_forward");
    TORCH_CHECK(query.dim() == 4 && key.dim() == 4 && value.dim() == 4,
                "paras sdpa_train_forward: [batch, heads, seq, head_dim] tensors");
    TORCH_CHECK(query.scalar_type() == c10::kBFloat16 || query.scalar_type() == c10::kHalf,
                "paras sdpa_train_forward: bfloat16 or float16 tensors");
    TORCH_CHECK(key.scalar_type() == query.scalar_type() && value.scalar_type() == query.scalar_type(),
                "paras sdpa_train_forward: query, key and value must have the same dtype");
    TORCH_CHECK(key.sizes() == value.sizes() && key.size(0) == query.size(0) && key.size(3) == query.size(3) &&
                    key.size(1) > 0 && query.size(1) % key.size(1) == 0,
                "paras sdpa_train_forward: shapes do not fit (query heads must be a multiple of key/value heads)");
    Runtime& rt = Runtime::get();
    c10::DeviceGuard guard(query.device());
    Tensor q = query.contiguous(), k = key.contiguous(), v = value.contiguous();
    const int64_t B = q.size(0), Hq = q.size(1), Lq = q.size(2), E = q.size(3);
    Tensor out = at::empty_like(q);
    Tensor lse = at::empty({B, Hq, Lq}, q.options().dtype(c10::kFloat));
    paras_sdpa_args a{};
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.out = out.data_ptr();
    a.lse = lse.numel() ? lse.data_ptr<float>() : nullptr;
    a.dtype = dtype_code(q.scalar_type());
    a.B = int32_t(B); a.Hq = int32_t(Hq); a.Hkv = int32_t(k.size(1));
    a.Lq = int32_t(Lq); a.Lk = int32_t(k.size(2)); a.D = int32_t(E);
    for (int i = 0; i < 3; ++i) {
        a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i);
        a.v_strides[i] = v.stride(i); a.o_strides[i] = out.stride(i);
    }
    a.causal = is_causal ? 1 : 0;
    a.scale = scale.has_value() ? *scale : 1.0 / std::sqrt(double(E));
    a.flags = ref_scale_rounding() ? PARAS_SDPA_REF_SCALE : 0;
    a.gpu = rt.gpu_of(query);
    PARAS_ABI(paras_b200_sdpa_fwd(&a));
    return {out, lse};
}

std::tuple<Tensor, Tensor, Tensor> sdpa_backward(const Tensor& grad_out, const Tensor& query, const Tensor& key,
                                                 const Tensor& value, const Tensor& out, const Tensor& lse,
                                                 bool is_causal, std::optional<double> scale) {
    PARAS_TRACE_OP("paras::sdpa_backward");
    TORCH_CHECK(query.dim() == 4 && key.dim() == 4 && value.dim() == 4 && grad_out.sizes() == query.sizes() &&
                    out.sizes() == query.sizes() && key.sizes() == value.sizes(),
                "paras sdpa_backward: shape mismatch");
    TORCH_CHECK(lse.scalar_type() == c10::kFloat && lse.numel() == query.numel() / std::max<int64_t>(query.size(3), 1),
                "paras sdpa_backward: lse must be the float32 [batch, heads, seq] tensor of the forward pass");
    Runtime& rt = Runtime::get();
    c10::DeviceGuard guard(query.device());
    Tensor q = query.contiguous(), k = key.contiguous(), v = value.contiguous();
    Tensor o = out.contiguous(), go = grad_out.contiguous(), l = lse.contiguous();
    Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
    paras_sdpa_bwd_args a{};
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.out = o.data_ptr(); a.dout = go.data_ptr();
    a.lse = l.numel() ? l.data_ptr<float>() : nullptr;
    a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
    a.B = int32_t(q.size(0)); a.Hq = int32_t(q.size(1)); a.Hkv = int32_t(k.size(1));
    a.Lq = int32_t(q.size(2)); a.Lk = int32_t(k.size(2)); a.D = int32_t(q.size(3));
    a.dtype = dtype_code(q.scalar_type());
    a.causal = is_causal ? 1 : 0;
    double sc = scale.has_value() ? *scale : 1.0 / std::sqrt(double(q.size(3)));
    if (ref_scale_rounding())  // the forward pass rounded the scale to the tensor dtype
        sc = at::scalar_tensor(sc, at::TensorOptions().dtype(q.scalar_type())).item<double>();
    a.scale = sc;
    a.gpu = rt.gpu_of(query);
    PARAS_ABI(paras_b200_sdpa_bwd(&a));
    return {dq, dk, dv};
}

// ---- rotary embedding fused into the attention prologue ----------------------------------------
// paras::sdpa_rope(q, k, v, cos, sin, is_causal, scale, q_pos0) = sdpa(rope(q), rope(k), v) with
// rope(x) = x * cos + rotate_half(x) * sin -- the composition a model builds from paras::rotate_half
// (fused_ops.cpp:234-267) and the reference's mul / add in front of its attention.  New operators
// (forward only); [batch, heads, seq, head_dim] tensors, cos / sin [positions, head_dim].
Tensor sdpa_rope(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& cos, const Tensor& sin,
                 bool is_causal, std::optional<double> scale, int64_t q_pos0) {
    PARAS_TRACE_OP("paras::sdpa_rope");
    TORCH_CHECK(query.dim() == 4 && key.dim() == 4 && value.dim() == 4,
                "paras sdpa_rope: [batch, heads, seq, head_dim] tensors");
    const int dt = dtype_code(query.scalar_type());
    TORCH_CHECK(dt >= 0 && key.scalar_type() == query.scalar_type() && value.scalar_type() == query.scalar_type() &&
                    cos.scalar_type() == query.scalar_type() && sin.scalar_type() == query.scalar_type(),
                "paras sdpa_rope: query, key, value, cos and sin must share one of float32, bfloat16, float16");
    const int64_t B = query.size(0), Hq = query.size(1), Lq = query.size(2), E = query.size(3);
    const int64_t Hkv = key.size(1), Lk = key.size(2);
    TORCH_CHECK(key.size(0) == B && value.sizes() == key.sizes() && key.size(3) == E && Hkv > 0 && Hq % Hkv == 0,
                "paras sdpa_rope: shapes do not fit (query heads must be a multiple of key/value heads)");
    TORCH_CHECK(cos.dim() == 2 && cos.size(1) == E && sin.sizes() == cos.sizes(),
                "paras sdpa_rope: cos and sin must be [positions, head_dim]");
    TORCH_CHECK(q_pos0 >= 0 && q_pos0 + Lq <= cos.size(0) && Lk <= cos.size(0),
                "paras sdpa_rope: cos / sin cover ", cos.size(0), " positions, fewer than the sequence needs");
    Runtime& rt = Runtime::get();
    c10::DeviceGuard guard(query.device());
    auto unit = [](const Tensor& t) { return (t.size(-1) > 1 && t.stride(-1) != 1) ? t.contiguous() : t; };
    Tensor q = unit(query), k = unit(key), v = unit(value), c = cos.contiguous(), sn = sin.contiguous();
    Tensor out = at::empty({B, Hq, Lq, E}, q.options());
    paras_sdpa_args a{};
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.out = out.data_ptr();
    a.dtype = dt;
    a.B = int32_t(B); a.Hq = int32_t(Hq); a.Hkv = int32_t(Hkv); a.Lq = int32_t(Lq); a.Lk = int32_t(Lk); a.D = int32_t(E);
    for (int i = 0; i < 3; ++i) {
        a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i);
        a.v_strides[i] = v.stride(i); a.o_strides[i] = out.stride(i);
    }
    a.causal = is_causal ? 1 : 0;
    a.scale = scale.has_value() ? *scale : 1.0 / std::sqrt(double(E));
    a.flags = ref_scale_rounding() ? PARAS_SDPA_REF_SCALE : 0;
    a.gpu = rt.gpu_of(query);
    PARAS_ABI(paras_b200_sdpa_rope_fwd(&a, c.data_ptr(), sn.data_ptr(), c.size(0), q_pos0));
    return out;
}

Tensor rope(const Tensor& x, const Tensor& cos, const Tensor& sin, int64_t pos0) {
    PARAS_TRACE_OP("paras::rope");
    TORCH_CHECK(x.dim() == 4, "paras rope: [batch, heads, seq, head_dim] tensor");
    const int dt = dtype_code(x.scalar_type());
    TORCH_CHECK(dt >= 0 && cos.scalar_type() == x.scalar_type() && sin.scalar_type() == x.scalar_type(),
                "paras rope: x, cos and sin must share one of float32, bfloat16, float16");
    TORCH_CHECK(x.size(3) % 2 == 0, "paras rope: last dimension must be even");
    TORCH_CHECK(cos.dim() == 2 && cos.size(1) == x.size(3) && sin.sizes() == cos.sizes() && pos0 >= 0 &&
                    pos0 + x.size(2) <= cos.size(0),
                "paras rope: cos and sin must be [positions, head_dim] and cover the sequence");
    c10::DeviceGuard guard(x.device());
    Tensor xs = (x.size(-1) > 1 && x.stride(-1) != 1) ? x.contiguous() : x;
    Tensor c = cos.contiguous(), sn = sin.contiguous();
    Tensor out = at::empty(x.sizes(), x.options());
    const int64_t st[3] = {xs.stride(0), xs.stride(1), xs.stride(2)};
    PARAS_ABI(paras_b200_rope(Runtime::get().gpu_of(x), xs.data_ptr(), st, c.data_ptr(), sn.data_ptr(), out.data_ptr(),
                              int(x.size(0)), int(x.size(1)), int(x.size(2)), int(x.size(3)), pos0, dt, nullptr));
    return out;
}

// ---- autograd for F.scaled_dot_product_attention on `paras` tensors ----------------------
// The reference's sdpa_math is built from at:: operators, so autograd differentiates through it
// (attention_ops.cpp:71-136).  A fused kernel registered for the backend replaces that
// composite for the autograd key too, so the gradient has to be tied on explicitly: when any of
// q, k, v requires grad the call goes to the differentiable pair sdpa_train_forward /
// sdpa_backward; what that pair does not cover raises instead of returning a result without a
// grad_fn.
struct SdpaFunction : public torch::autograd::Function<SdpaFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& q, const Tensor& k,
                          const Tensor& v, bool is_causal, std::optional<double> scale) {
        auto [out, lse] = sdpa_train_forward(q, k, v, is_causal, scale);
        ctx->save_for_backward({q, k, v, out, lse});
        ctx->saved_data["is_causal"] = is_causal;
        ctx->saved_data["has_scale"] = scale.has_value();
        ctx->saved_data["scale"] = scale.value_or(0.0);
        return out;
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grads) {
        const auto saved = ctx->get_saved_variables();
        std::optional<double> scale;
        if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
        auto [dq, dk, dv] = sdpa_backward(grads[0], saved[0], saved[1], saved[2], saved[3], saved[4],
                                          ctx->saved_data["is_causal"].toBool(), scale);
        return {dq, dk, dv, Tensor(), Tensor()};
    }
};

// Everything the fused pair does not take (an attn_mask, dropout, fp32, other head dims): the forward
// the operator would run anyway, and the CUDA-core backward of exactly that call, with the forward's
// dropout counters replayed.
struct SdpaGeneralFunction : public torch::autograd::Function<SdpaGeneralFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& q, const Tensor& k, const Tensor& v,
                          const std::optional<Tensor>& mask, double dropout_p, bool is_causal,
                          std::optional<double> scale, bool enable_gqa) {
        RngState rng{0, 0};
        const bool has_mask = mask.has_value() && mask->defined();
        Tensor out = sdpa_forward(q, k, v, mask, dropout_p, is_causal, scale, enable_gqa, std::nullopt, nullptr, &rng);
        if (has_mask) ctx->save_for_backward({q, k, v, *mask});
        else ctx->save_for_backward({q, k, v});
        ctx->saved_data["has_mask"] = has_mask;
        ctx->saved_data["dropout_p"] = dropout_p;
        ctx->saved_data["is_causal"] = is_causal;
        ctx->saved_data["has_scale"] = scale.has_value();
        ctx->saved_data["scale"] = scale.value_or(0.0);
        ctx->saved_data["enable_gqa"] = enable_gqa;
        ctx->saved_data["seed"] = static_cast<int64_t>(rng.first);
        ctx->saved_data["sequence"] = static_cast<int64_t>(rng.second);
        return out;
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grads) {
        const auto saved = ctx->get_saved_variables();
        std::optional<double> scale;
        if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
        std::optional<Tensor> m;
        if (ctx->saved_data["has_mask"].toBool()) m = saved[3];
        const RngState rng{static_cast<uint64_t>(ctx->saved_data["seed"].toInt()),
                           static_cast<uint64_t>(ctx->saved_data["sequence"].toInt())};
        Tensor go = grads[0].contiguous();
        GradRequest req{&go, &rng, Tensor(), Tensor(), Tensor()};
        sdpa_forward(saved[0], saved[1], saved[2], m, ctx->saved_data["dropout_p"].toDouble(),
                     ctx->saved_data["is_causal"].toBool(), scale, ctx->saved_data["enable_gqa"].toBool(),
                     std::nullopt, nullptr, nullptr, &req);
        return {req.dq, req.dk, req.dv, Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

// Is `mask` one [Lq, Lk] mask for every batch element and head, and the causal mask written out?  Then the call
// is the reference's is_causal=True (attention_ops.cpp:100-116 builds exactly that mask) and can take the fused
// kernels, whose backward takes no mask tensor.  The answer needs a pass over the mask on the GPU and a wait for
// it, so it is remembered for the tensor (storage, version, shape): a model hands the same mask to every layer.
bool mask_is_causal(const Tensor& mask, const Tensor& query, int64_t Lq, int64_t Lk, double scale) {
    if (mask.dim() < 2 || mask.size(-2) != Lq || mask.size(-1) != Lk || mask.stride(-1) != 1 || Lq < 2 || Lk < 2) return false;
    for (int64_t d = 0; d + 2 < mask.dim(); ++d)
        if (mask.size(d) != 1) return false;
    int kind;
    if (mask.scalar_type() == c10::kBool) kind = 1;
    else if (mask.scalar_type() == query.scalar_type()) kind = 2;
    else if (mask.scalar_type() == c10::kFloat) kind = 3;
    else return false;
    // The remembered mask is held, so that its memory cannot be handed to another tensor while the answer is
    // kept; a write to it moves its version.  (Heap-allocated and never destroyed: a tensor of this device
    // must not be released during static destruction, after the runtime.)
    struct Seen { Tensor held; const void* ptr; uint32_t version; int64_t Lq, Lk, stride; int kind; double scale; bool result; };
    static thread_local Seen& seen = *new Seen{Tensor(), nullptr, 0, 0, 0, 0, 0, 0.0, false};
    const void* ptr = mask.data_ptr();
    const bool tracked = !mask.is_inference();     // an inference tensor has no version counter: ask every time
    const uint32_t version = tracked ? mask._version() : 0;
    if (tracked && seen.held.defined() && seen.ptr == ptr && seen.version == version && seen.Lq == Lq && seen.Lk == Lk &&
        seen.stride == mask.stride(-2) && seen.kind == kind && seen.scale == scale)
        return seen.result;
    Runtime& rt = Runtime::get();
    c10::DeviceGuard guard(query.device());
    int result = 0;
    PARAS_ABI(paras_b200_sdpa_mask_is_causal(rt.gpu_of(query), ptr, kind, dtype_code(query.scalar_type()), mask.stride(-2),
                                             int32_t(Lq), int32_t(Lk), scale, nullptr, &result));
    if (tracked) seen = Seen{mask, ptr, version, Lq, Lk, mask.stride(-2), kind, scale, result != 0};
    return result != 0;
}

Tensor sdpa_autograd(const Tensor& query, const Tensor& key, const Tensor& value,
                     const std::optional<Tensor>& attn_mask_in, double dropout_p, bool is_causal_in,
                     std::optional<double> scale, bool enable_gqa) {
    std::optional<Tensor> attn_mask = attn_mask_in;
    bool is_causal = is_causal_in;
    const bool needs_grad = at::GradMode::is_enabled() &&
                            (query.requires_grad() || key.requires_grad() || value.requires_grad());
    if (!needs_grad) {
        at::AutoDispatchBelowADInplaceOrView below;
        return at::scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale,
                                                enable_gqa);
    }
    bool has_mask = attn_mask.has_value() && attn_mask->defined();
    TORCH_CHECK(query.dim() >= 3 && key.dim() == query.dim() && value.dim() == query.dim(),
                "paras sdpa: query, key and value must have the same rank (>= 3)");
    // the fused kernels: 16-bit, no mask tensor, no dropout, head dim 128 / 64 (or, on the composite of
    // GEMMs, 16-byte rows of both the head dim and the key length)
    const int64_t E = query.size(-1), Lk = key.size(-2);
    const bool half = query.scalar_type() == c10::kBFloat16 || query.scalar_type() == c10::kHalf;
    // a causal mask passed as a tensor is is_causal=True
    if (has_mask && !is_causal && dropout_p == 0.0 && half && (E == 128 || E == 64) && query.numel() > 0 && key.numel() > 0 &&
        attn_mask->device() == query.device() &&
        mask_is_causal(*attn_mask, query, query.size(-2), Lk, scale.has_value() ? *scale : 1.0 / std::sqrt(double(E)))) {
        has_mask = false;
        is_causal = true;
        attn_mask = std::nullopt;
    }
    const bool fused = !has_mask && dropout_p == 0.0 && half && E % 8 == 0 && (E == 128 || E == 64 || Lk % 8 == 0) &&
                       query.numel() > 0 && key.numel() > 0;
    if (!fused)
        return SdpaGeneralFunction::apply(query, key, value, has_mask ? attn_mask : std::optional<Tensor>(), dropout_p,
                                          is_causal, scale, enable_gqa);
    Tensor q = query, k = key, v = value;
    if (q.dim() == 3) { q = q.unsqueeze(1); k = k.unsqueeze(1); v = v.unsqueeze(1); }
    else if (q.dim() > 4) {
        q = q.reshape({-1, q.size(-3), q.size(-2), q.size(-1)});
        k = k.reshape({-1, k.size(-3), k.size(-2), k.size(-1)});
        v = v.reshape({-1, v.size(-3), v.size(-2), v.size(-1)});
    }
    TORCH_CHECK(k.size(1) == q.size(1) || enable_gqa, "paras sdpa: key/value have ", k.size(1),
                " heads but query has ", q.size(1), "; pass enable_gqa=True for grouped-query attention");
    Tensor out = SdpaFunction::apply(q, k, v, is_causal, scale);
    if (query.dim() == 3) return out.squeeze(1);
    if (query.dim() > 4) return out.reshape(query.sizes());
    return out;
}

}  // namespace
}  // namespace paras

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("aten::_scaled_dot_product_attention_math", &paras::sdpa_math);
    m.impl("aten::scaled_dot_product_attention", &paras::sdpa);
}
TORCH_LIBRARY_IMPL(aten, AutogradPrivateUse1, m) {
    m.impl("aten::scaled_dot_product_attention", &paras::sdpa_autograd);
}

TORCH_LIBRARY_FRAGMENT(paras, m) {
    m.def("sdpa_train_forward(Tensor query, Tensor key, Tensor value, bool is_causal, float? scale) -> (Tensor, Tensor)");
    m.def("sdpa_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value, Tensor out, Tensor lse, "
          "bool is_causal, float? scale) -> (Tensor, Tensor, Tensor)");
    m.def("sdpa_rope(Tensor query, Tensor key, Tensor value, Tensor cos, Tensor sin, bool is_causal, float? scale, "
          "int q_pos0=0) -> Tensor");
    m.def("rope(Tensor x, Tensor cos, Tensor sin, int pos0=0) -> Tensor");
}
TORCH_LIBRARY_IMPL(paras, PrivateUse1, m) {
    m.impl("sdpa_train_forward", &paras::sdpa_train_forward);
    m.impl("sdpa_backward", &paras::sdpa_backward);
    m.impl("sdpa_rope", &paras::sdpa_rope);
    m.impl("rope", &paras::rope);
}
