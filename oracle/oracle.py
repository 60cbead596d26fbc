"""CPU restatement of the reference's transformer hot path (the ORACLE).

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this file; only tests/,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg may.  It restates, with
plain torch-CPU / numpy arithmetic, what the reference's ``paras:0`` host engine computes
for scaled-dot-product attention, RMSNorm and SwiGLU, including where the reference
rounds intermediates to the tensor dtype.  Pinned against the real reference build
(oracle/_ref/_C.so run through oracle/ref_run.py): see tests/golden/make_golden.py and
tests/test_oracle_pins.py.

Reference files restated (paths inside the reference project):
  * csrc/ops/attention_ops.cpp:71-136      sdpa_math (composition)
  * csrc/ops/vision_ops.cpp:398-406        bmm.out  = libtorch CPU ``at::bmm`` on host copies
  * csrc/ops/pointwise_ops.cpp:62-85       binary_kernel: double math, result cast to dtype,
                                           a Python/C++ scalar operand is first materialised
                                           as a 0-dim tensor OF THE OUTPUT DTYPE (line 54-59)
  * csrc/ops/pointwise_ops.cpp:33-52       unary_kernel: double math, result cast to dtype
  * csrc/ops/pointwise_ops.cpp:926-981     softmax_out: per row max / sum exp / normalise in double
  * csrc/ops/scatter_ops.cpp:43-71         masked_fill_
  * csrc/ops/rms_swiglu_ops.cpp:43-86      aten::rms_norm and torch_paras::swiglu composites
  * csrc/ops/fused_ops.cpp:43-88,162-194   paras::rms_norm and paras::swiglu fused lambdas
  * csrc/ops/fused_ops.cpp:90-157,196-302  their backward ops and rotate_half

A C++ ``static_cast<scalar_t>(double)`` for bf16/fp16 goes double -> float -> 16-bit
(c10's 16-bit types construct from float), i.e. it rounds twice; ``_cast`` does the same.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

Tensor = torch.Tensor


def _cast(x64: Tensor, dtype: torch.dtype) -> Tensor:
    """double -> dtype the way ``static_cast<scalar_t>(double)`` does it."""
    if dtype == torch.float64:
        return x64
    x32 = x64.to(torch.float32)
    return x32 if dtype == torch.float32 else x32.to(dtype)


def _scalar_as(value: float, dtype: torch.dtype) -> float:
    """A scalar operand is wrapped into a 0-dim tensor of the output dtype before the
    kernel reads it back as double (pointwise_ops.cpp:54-59, 62-70)."""
    return float(_cast(torch.tensor(value, dtype=torch.float64), dtype).to(torch.float64))


def _seq_sum_lastdim(x64: Tensor) -> Tensor:
    """Left-to-right double accumulation over the last dim (the reference loops serially)."""
    return torch.from_numpy(np.cumsum(x64.numpy(), axis=-1)[..., -1].copy())


# ----------------------------------------------------------------------------------
# building blocks
# ----------------------------------------------------------------------------------
def mul_scalar(x: Tensor, s: float) -> Tensor:
    return _cast(x.to(torch.float64) * _scalar_as(s, x.dtype), x.dtype)


def softmax_lastdim(x: Tensor) -> Tensor:
    """pointwise_ops.cpp:954-977: three serial passes in double, output in input dtype."""
    x64 = x.to(torch.float64)
    m = x64.max(dim=-1, keepdim=True).values
    e = torch.exp(x64 - m)
    s = _seq_sum_lastdim(e).unsqueeze(-1)
    return _cast(e / s, x.dtype)


def matmul_ref(a: Tensor, b: Tensor) -> Tensor:
    """Upstream ``at::matmul`` folds the leading dims and calls ``bmm.out``; the reference's
    bmm_out makes CONTIGUOUS host copies of both operands and runs libtorch's CPU ``at::bmm``
    on them (vision_ops.cpp:34-36,398-406).  The result has the operands' dtype."""
    if a.dim() < 3 or b.dim() < 3 or a.shape[:-2] != b.shape[:-2]:
        return torch.matmul(a, b)
    lead = a.shape[:-2]
    a3 = a.reshape(-1, a.size(-2), a.size(-1)).contiguous()
    b3 = b.reshape(-1, b.size(-2), b.size(-1)).contiguous()
    return torch.bmm(a3, b3).reshape(*lead, a.size(-2), b.size(-1))


# ----------------------------------------------------------------------------------
# dropout  (random_ops.cpp:27-59 Philox2x32-10, 140-176 native_dropout; context.cpp:76-83)
# ----------------------------------------------------------------------------------
def philox2x32_r0(seed: int, sequence: int, n: int) -> np.ndarray:
    """First output word of Philox2x32-10 for counters 0..n-1 (random_ops.cpp:27-47): counter
    (idx low word, sequence + idx high word), key = seed's low word bumped by 0x9E3779B9 per round."""
    idx = np.arange(n, dtype=np.uint64)
    c0 = (idx & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = ((np.uint64(sequence) + (idx >> np.uint64(32))) & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    k0 = int(seed) & 0xFFFFFFFF
    m = np.uint64(0xD256D193)
    for _ in range(10):
        prod = m * c0                                   # both below 2^32: the product fits 64 bits
        n0 = ((prod >> np.uint64(32)) ^ np.uint64(k0) ^ c1) & np.uint64(0xFFFFFFFF)
        c1 = prod & np.uint64(0xFFFFFFFF)
        c0 = n0
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
    return c0.astype(np.uint32)


def rng_advance(sequence: int, items: int) -> int:
    """Context::rng_draw: the sequence after an operator that drew `items` numbers."""
    return sequence + (items + 1) // 2 + 1


def native_dropout(x: Tensor, p: float, seed: int, sequence: int) -> Tensor:
    """random_ops.cpp:140-176 on a contiguous tensor: element i is kept when
    (r0 >> 8) * 2^-24 < float(1 - p) and becomes dtype(float(x) * (1.0f / keep))."""
    keep = np.float32(1.0 - p)
    scale = np.float32(1.0) / keep
    r0 = philox2x32_r0(seed, sequence, x.numel())
    u = (r0 >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / (1 << 24))
    kept = torch.from_numpy(u < keep).reshape(x.shape)
    scaled = (x.contiguous().to(torch.float32) * float(scale)).to(x.dtype)
    return torch.where(kept, scaled, torch.zeros_like(scaled))


# ----------------------------------------------------------------------------------
# scaled dot product attention  (attention_ops.cpp:71-136)
# ----------------------------------------------------------------------------------
def sdpa(q: Tensor, k: Tensor, v: Tensor, attn_mask: Optional[Tensor] = None,
         is_causal: bool = False, scale: Optional[float] = None,
         enable_gqa: bool = False, return_weights: bool = False, dropout_p: float = 0.0,
         dropout_mask: Optional[Tensor] = None, rng: Tuple[int, int] = (0x5deece66d, 0)):
    """`rng` = (seed, sequence) of the device when the call is made; the weights returned are the
    ones after dropout, as the reference returns them (attention_ops.cpp:128-135)."""
    if q.dim() < 3 or k.dim() < 3 or v.dim() < 3:
        raise RuntimeError("paras sdpa: query/key/value must be at least 3-D")
    if is_causal and attn_mask is not None:
        raise RuntimeError("paras sdpa: is_causal and attn_mask are mutually exclusive")
    if enable_gqa and k.size(-3) != q.size(-3):
        if q.size(-3) % k.size(-3) != 0:
            raise RuntimeError("paras sdpa: query heads must be a multiple of key/value heads")
        rep = q.size(-3) // k.size(-3)
        k = k.repeat_interleave(rep, dim=-3)
        v = v.repeat_interleave(rep, dim=-3)
    d = q.size(-1)
    scale_factor = scale if scale is not None else 1.0 / math.sqrt(float(d))
    scores = mul_scalar(matmul_ref(q, k.transpose(-2, -1)), scale_factor)
    lq, lk = q.size(-2), k.size(-2)
    if is_causal:
        # tril(ones(Lq, Lk), 0): query i sees keys 0..i whatever Lk - Lq is (103-116)
        allow = torch.ones(lq, lk, dtype=torch.bool).tril(0)
        scores = scores.masked_fill(~allow, float("-inf"))
    elif attn_mask is not None:
        if attn_mask.dtype == torch.bool:
            scores = scores.masked_fill(~attn_mask, float("-inf"))
        else:
            out_dtype = torch.result_type(scores, attn_mask)
            scores = _cast(scores.to(torch.float64) + attn_mask.to(torch.float64), out_dtype)
    attn = softmax_lastdim(scores)
    if dropout_p > 0.0:
        if dropout_mask is not None:      # attn * mask / (1 - p): two binary kernels, each rounding
            dt = torch.result_type(attn, dropout_mask)
            attn = _cast(attn.to(torch.float64) * dropout_mask.to(torch.float64), dt)
            attn = _cast(attn.to(torch.float64) / _scalar_as(1.0 - dropout_p, dt), dt)
        else:                             # at::dropout -> native_dropout on the device
            attn = native_dropout(attn, dropout_p, rng[0], rng[1])
    out = matmul_ref(attn, v)
    return (out, attn) if return_weights else out


# ----------------------------------------------------------------------------------
# RMSNorm
# ----------------------------------------------------------------------------------
def rms_norm_composite(x: Tensor, normalized_shape: Sequence[int],
                       weight: Optional[Tensor] = None, eps: Optional[float] = None) -> Tensor:
    """aten::rms_norm on the reference (rms_swiglu_ops.cpp:43-75): every step rounds to the
    tensor dtype -- pow, sum, *1/N, +eps, rsqrt, *inv, *weight."""
    nd = len(normalized_shape)
    if nd < 1:
        raise RuntimeError("paras rms_norm: normalized_shape must be non-empty")
    if x.dim() < nd or tuple(x.shape[x.dim() - nd:]) != tuple(normalized_shape):
        raise RuntimeError("paras rms_norm: normalized_shape does not match the trailing dims")
    if weight is not None and tuple(weight.shape) != tuple(normalized_shape):
        raise RuntimeError("paras rms_norm: weight shape must equal normalized_shape")
    dt = x.dtype
    eps_val = 1e-6 if eps is None else eps
    lead = x.shape[: x.dim() - nd]
    n = 1
    for s in normalized_shape:
        n *= int(s)
    x64 = x.to(torch.float64)
    sq = _cast(torch.pow(x64, 2.0), dt)                                     # pow.Tensor_Scalar_out
    ssum = _cast(_seq_sum_lastdim(sq.reshape(*lead, n).to(torch.float64)), dt)   # reduce_outer
    mean = _cast(ssum.to(torch.float64) * (1.0 / float(n)), dt)             # post_scale pass
    mean = _cast(mean.to(torch.float64) + _scalar_as(eps_val, dt), dt)      # add.out
    inv = _cast(1.0 / torch.sqrt(mean.to(torch.float64)), dt)               # rsqrt.out
    inv = inv.reshape(*lead, *([1] * nd))
    out = _cast(x64 * inv.to(torch.float64), dt)                            # mul.out
    if weight is not None:
        out = _cast(out.to(torch.float64) * weight.to(torch.float64), dt)   # mul.out
    return out


def rms_norm_fused(x: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    """paras::rms_norm (fused_ops.cpp:43-88): last dim only, double math, one rounding;
    also returns rstd[rows] in fp32."""
    h = x.size(-1)
    if weight.numel() != h:
        raise RuntimeError("paras rms_norm: weight size must match the last dimension")
    x64 = x.contiguous().to(torch.float64)
    rows = x64.numel() // h if h > 0 else 0
    x2 = x64.reshape(rows, h)
    ss = _seq_sum_lastdim(x2 * x2) if rows and h else torch.zeros(rows, dtype=torch.float64)
    rms = 1.0 / torch.sqrt(ss / float(h) + eps)
    out = _cast((x2 * rms.unsqueeze(-1)) * weight.contiguous().to(torch.float64).reshape(1, h),
                x.dtype).reshape(x.shape)
    return out, rms.to(torch.float32)


def rms_norm_fused_backward(grad_out: Tensor, x: Tensor, weight: Tensor,
                            rstd: Tensor) -> Tuple[Tensor, Tensor]:
    """paras::rms_norm_backward (fused_ops.cpp:90-157)."""
    h = x.size(-1)
    rows = x.numel() // h if h > 0 else 0
    g = grad_out.contiguous().to(torch.float64).reshape(rows, h)
    xx = x.contiguous().to(torch.float64).reshape(rows, h)
    w = weight.contiguous().to(torch.float64).reshape(1, h)
    rr = rstd.to(torch.float64).reshape(rows, 1)
    dot = _seq_sum_lastdim(g * w * xx).unsqueeze(-1)
    coef = rr * rr * rr / float(h)
    gi = _cast(g * w * rr - coef * xx * dot, x.dtype).reshape(x.shape)
    gw64 = torch.from_numpy(np.cumsum((g * xx * rr).numpy(), axis=0)[-1].copy()) if rows else \
        torch.zeros(h, dtype=torch.float64)
    return gi, _cast(gw64, weight.dtype)


# ----------------------------------------------------------------------------------
# SwiGLU
# ----------------------------------------------------------------------------------
def swiglu_fused(gate: Tensor, up: Tensor) -> Tensor:
    """paras::swiglu(gate, up) (fused_ops.cpp:162-194): g/(1+exp(-g))*u in double, one rounding."""
    if gate.shape != up.shape:
        raise RuntimeError("paras swiglu: gate and up must have the same shape")
    g = gate.to(torch.float64)
    return _cast((g / (1.0 + torch.exp(-g))) * up.to(torch.float64), gate.dtype)


def swiglu_fused_backward(grad_out: Tensor, gate: Tensor, up: Tensor) -> Tuple[Tensor, Tensor]:
    """paras::swiglu_backward (fused_ops.cpp:196-229)."""
    dy = grad_out.to(torch.float64)
    g = gate.to(torch.float64)
    u = up.to(torch.float64)
    s = 1.0 / (1.0 + torch.exp(-g))
    return (_cast(dy * u * (s * (1.0 + g * (1.0 - s))), gate.dtype),
            _cast(dy * g * s, up.dtype))


def swiglu_composite(x: Tensor, gate: Tensor) -> Tensor:
    """torch_paras::swiglu(x, gate) = x * silu(gate) (rms_swiglu_ops.cpp:83-86); silu's result
    is rounded to the dtype before the multiply (pointwise_ops.cpp:460-464)."""
    g = gate.to(torch.float64)
    silu = _cast(g / (1.0 + torch.exp(-g)), gate.dtype)
    dt = torch.result_type(x, silu)
    return _cast(x.to(torch.float64) * silu.to(torch.float64), dt)


def rotate_half(x: Tensor) -> Tensor:
    """paras::rotate_half (fused_ops.cpp:234-267): cat(-x2, x1) over the last dim."""
    d = x.size(-1)
    if d % 2:
        raise RuntimeError("paras rotate_half: last dimension must be even")
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope(x: Tensor, cos: Tensor, sin: Tensor, pos0: int = 0) -> Tensor:
    """Rotary embedding as a user of the reference composes it from its operators:
    x * cos + rotate_half(x) * sin, with x [..., L, D] and cos/sin [Lmax, D] rows pos0 .. pos0+L-1;
    each of the two products and the sum is a binary kernel that rounds to the tensor dtype
    (pointwise_ops.cpp:62-85), rotate_half is exact (fused_ops.cpp:234-267)."""
    L = x.size(-2)
    c, sn = cos[pos0:pos0 + L].to(torch.float64), sin[pos0:pos0 + L].to(torch.float64)
    t1 = _cast(x.to(torch.float64) * c, x.dtype)
    t2 = _cast(rotate_half(x).to(torch.float64) * sn, x.dtype)
    return _cast(t1.to(torch.float64) + t2.to(torch.float64), x.dtype)


def rotate_half_backward(g: Tensor) -> Tensor:
    """paras::rotate_half_backward (fused_ops.cpp:269-302): cat(g2, -g1)."""
    d = g.size(-1)
    g1, g2 = g[..., : d // 2], g[..., d // 2:]
    return torch.cat((g2, -g1), dim=-1)


# ----------------------------------------------------------------------------------
# matrix products either side of the path: the reference hands them to libtorch on the host
# ----------------------------------------------------------------------------------
def mm(a: Tensor, b: Tensor) -> Tensor:
    """mm_out (vision_ops.cpp:388-396): at::mm on host copies of both operands."""
    return torch.mm(a.contiguous(), b.contiguous())


def bmm(a: Tensor, b: Tensor) -> Tensor:
    """bmm_out (vision_ops.cpp:398-406): at::bmm on host copies."""
    return torch.bmm(a.contiguous(), b.contiguous())


def addmm(c: Tensor, a: Tensor, b: Tensor, beta=1, alpha=1) -> Tensor:
    """addmm_out (vision_ops.cpp:408-423): at::addmm on host copies."""
    return torch.addmm(c, a.contiguous(), b.contiguous(), beta=beta, alpha=alpha)


def linear(x: Tensor, w: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """LinearFunction::forward (vision_ops.cpp:248-270): at::linear on host copies."""
    return torch.nn.functional.linear(x, w, bias)


def swiglu_linear(x: Tensor, w_gate: Tensor, w_up: Tensor) -> Tensor:
    """What the reference computes for a gated MLP's first half: two linear calls, each rounded
    to the tensor dtype, then paras::swiglu (fused_ops.cpp:162-194)."""
    return swiglu_fused(linear(x, w_gate), linear(x, w_up))


# ----------------------------------------------------------------------------------
# synthetic inputs of the five benchmark configurations
# ----------------------------------------------------------------------------------
def gen_seed(config_index: int, batch: Optional[int] = None) -> int:
    base = 1000 + config_index
    return base if batch is None else base * 10 ** 6 + batch


def randn(shape, gen: torch.Generator, dtype=torch.float32, mean=0.0, std=1.0) -> Tensor:
    t = torch.randn(shape, generator=gen, dtype=torch.float32)
    if mean != 0.0 or std != 1.0:
        t = mean + std * t
    return t.to(dtype)
