"""Differentiable wrappers over the fused ``paras::`` operators.

Same public functions as the reference's python/torch_paras/nn.py:36-89 (``rms_norm``,
``swiglu``, ``rotate_half``): a custom-op namespace has no autograd formula of its own, so
each forward/backward pair is tied together with a ``torch.autograd.Function``.
"""
import torch

from . import _C  # noqa: F401  (loads the operator registrations)

__all__ = ["rms_norm", "swiglu", "rotate_half", "rope", "attention_rope", "swiglu_linear", "rms_norm_linear",
           "fold_norm_weight",
           "attention_host", "scaled_dot_product_attention"]


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        out, rstd = torch.ops.paras.rms_norm(x, weight, eps)
        ctx.save_for_backward(x, weight, rstd)
        return out

    @staticmethod
    def backward(ctx, grad):
        x, weight, rstd = ctx.saved_tensors
        gx, gw = torch.ops.paras.rms_norm_backward(grad.contiguous(), x, weight, rstd)
        return gx, gw, None


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return torch.ops.paras.swiglu(gate, up)

    @staticmethod
    def backward(ctx, grad):
        gate, up = ctx.saved_tensors
        return torch.ops.paras.swiglu_backward(grad.contiguous(), gate, up)


class _SDPA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal, scale):
        out, lse = torch.ops.paras.sdpa_train_forward(q, k, v, is_causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.is_causal, ctx.scale = is_causal, scale
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.ops.paras.sdpa_backward(grad.contiguous(), q, k, v, out, lse,
                                                   ctx.is_causal, ctx.scale)
        return dq, dk, dv, None, None


class _RotateHalf(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return torch.ops.paras.rotate_half(x)

    @staticmethod
    def backward(ctx, grad):
        return torch.ops.paras.rotate_half_backward(grad.contiguous())


def rms_norm(input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the last dimension of ``input`` in one kernel."""
    return _RMSNorm.apply(input, weight, eps)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` in one kernel."""
    return _SwiGLU.apply(gate, up)


def swiglu_linear(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``swiglu(F.linear(x, w_gate), F.linear(x, w_up))`` as one GEMM kernel (forward only):
    both projections share one pass over ``x`` and SwiGLU runs in the epilogue.  16-bit
    operands; the weights are ``[features, in_features]`` like ``nn.Linear.weight``."""
    return torch.ops.paras.swiglu_linear(x, w_gate, w_up)


def fold_norm_weight(weight: torch.Tensor, norm_weight: torch.Tensor) -> torch.Tensor:
    """``weight * norm_weight`` (broadcast over rows): the RMSNorm weight moved into the ``[out, in]``
    weight of the projection that follows the norm.  Do it once per weight and pass the result to
    ``rms_norm_linear(..., folded_weight=...)``."""
    return torch.ops.paras.fold_norm_weight(weight, norm_weight)


def rms_norm_linear(x: torch.Tensor, norm_weight: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *,
                    folded_weight: torch.Tensor = None) -> torch.Tensor:
    """``F.linear(rms_norm(x, norm_weight, eps), weight)`` (forward only, 16-bit) without the normalised
    activations ever being written: one read of ``x`` for the row statistic, then the projection GEMM
    whose epilogue scales each output row by it."""
    if folded_weight is not None:
        return torch.ops.paras.rms_norm_linear_folded(x, folded_weight, eps)
    return torch.ops.paras.rms_norm_linear(x, norm_weight, weight, eps)


def attention_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *,
                   is_causal: bool = False, scale=None, out=None, device: int = 1) -> torch.Tensor:
    """Scaled dot-product attention for operands that live on the HOST ([B, H, L, D], 16-bit
    or fp32, GQA by head count): batch chunks stream through GPU ``paras:device`` -- copy in,
    attention, copy out, the three overlapping -- and the result is returned as a host tensor
    (page-locked unless ``out`` is given).  Same numerics as
    ``F.scaled_dot_product_attention`` on the ``paras`` device; use it instead of
    ``.to("paras:N")`` + attention + ``.cpu()`` when the data does not stay on the GPU.
    Pass ``pin_memory()``-ed tensors: pageable ones are staged and lose most of the overlap."""
    from . import abi
    if device < 1:
        raise RuntimeError("paras attention_host: device must be a GPU index (paras:1 and up)")
    return abi.sdpa_fwd_host(query.contiguous(), key.contiguous(), value.contiguous(),
                             causal=is_causal, scale=scale, flags=abi.SDPA_REF_SCALE, out=out,
                             gpu=device - 1)


def scaled_dot_product_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *,
                                 is_causal: bool = False, scale=None) -> torch.Tensor:
    """Differentiable attention on ``paras`` tensors ([batch, heads, seq, head_dim], bfloat16 or
    float16, fewer key/value heads than query heads = GQA).  Forward is the fused kernel (it also
    keeps each row's log-sum-exp); backward rebuilds the probabilities from it and runs as five
    batched GEMMs and two element-wise passes.  ``F.scaled_dot_product_attention`` on the device is
    the inference entry point (forward only, masks, any rank)."""
    return _SDPA.apply(query, key, value, is_causal, scale)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos0: int = 0) -> torch.Tensor:
    """Rotary embedding ``x * cos + rotate_half(x) * sin`` in one kernel (forward only): ``x`` is
    ``[batch, heads, seq, head_dim]``, ``cos`` / ``sin`` ``[positions, head_dim]`` read from row ``pos0``."""
    return torch.ops.paras.rope(x, cos, sin, pos0)


def attention_rope(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, cos: torch.Tensor,
                   sin: torch.Tensor, *, is_causal: bool = False, scale=None, q_pos0: int = 0) -> torch.Tensor:
    """``scaled_dot_product_attention(rope(query), rope(key), value)`` (forward only) without the rotated
    queries ever reaching memory: with 16-bit tensors and head dim 128 they are rotated inside the
    attention kernel; the keys are rotated once, on the way in."""
    return torch.ops.paras.sdpa_rope(query, key, value, cos, sin, is_causal, scale, q_pos0)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """RoPE helper ``cat(-x2, x1, dim=-1)`` with ``x1, x2 = x.chunk(2, dim=-1)``."""
    return _RotateHalf.apply(x)
