"""Attention backward (paras_b200_sdpa_bwd, torch_paras.nn.scaled_dot_product_attention) against
the gradient of float64 attention on the same 16-bit inputs.

The reference differentiates through its composite attention with 16-bit intermediates
(scores, probabilities and their gradients are all rounded, csrc/ops/attention_ops.cpp:96-135,
pointwise_ops.cpp:994-1062); this implementation rounds the same four [L, L] matrices.  The
tolerance is therefore relative to each gradient's scale: max |got - want| <= 3e-2 * max |want|
and a mean error below 1 % of it.
"""
import math

import pytest
import torch
import torch.nn.functional as F

import torch_paras
from torch_paras import abi, nn as paras_nn

pytestmark = pytest.mark.gpu
CUDA = "cuda:0"
DEV = "paras:1"


def reference_grads(q, k, v, dout, causal):
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    r = q.shape[1] // k.shape[1]
    kk, vv = k64.repeat_interleave(r, 1), v64.repeat_interleave(r, 1)
    s = (q64 @ kk.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if causal:
        Lq, Lk = q.shape[2], k.shape[2]
        s = s.masked_fill(~torch.ones(Lq, Lk, dtype=torch.bool).tril(), float("-inf"))
    out = torch.softmax(s, -1) @ vv
    out.backward(dout.double())
    return q64.grad, k64.grad, v64.grad


def check(got, want, name):
    got = got.detach().cpu().double()
    scale = want.abs().max().item()
    err = (got - want).abs()
    assert torch.isfinite(got).all(), name
    assert err.max().item() <= 3e-2 * scale, f"{name}: max error {err.max().item():.3e} vs scale {scale:.3e}"
    assert err.mean().item() <= 1e-2 * scale, f"{name}: mean error {err.mean().item():.3e} vs scale {scale:.3e}"


CASES = [
    # B, Hq, Hkv, Lq, Lk, D, causal
    (1, 2, 2, 256, 256, 128, True),
    (2, 4, 2, 384, 384, 128, True),      # GQA: dk / dv sum over the group's query heads
    (1, 4, 1, 200, 328, 128, False),     # ragged rows, Lq != Lk
    (1, 2, 2, 136, 264, 64, True),       # D = 64, top-left aligned causal mask with Lk > Lq
    (1, 4, 2, 1000, 1000, 128, True),    # stacked heads whose 128-row tiles straddle two heads
    (1, 2, 2, 640, 320, 128, True),      # fewer keys than queries
    (2, 2, 1, 1024, 1024, 64, True),     # several causally empty 128 x 256 tiles per head
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_backward_through_the_c_abi(case, dtype):
    B, Hq, Hkv, Lq, Lk, D, causal = case
    g = torch.Generator().manual_seed(41)
    q = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
    dout = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
    qd, kd, vd, dd = (t.to(CUDA) for t in (q, k, v, dout))
    out, lse = abi.sdpa_fwd(qd, kd, vd, causal=causal, return_lse=True)
    # Causally empty tiles of the two [rows, Lk] scratch matrices are never written and must never be
    # read: fill the library's pool with NaN first, so that a read of one would show in the gradients.
    scratch = B * Hq * Lq * 4 + 2 * B * Hq * Lq * Lk * 2 + 4096
    poison = torch.full((scratch // 4,), float("nan"), dtype=torch.float32, device=DEV)
    torch_paras.synchronize()
    del poison
    dq, dk, dv = abi.sdpa_bwd(dd, qd, kd, vd, out, lse, causal=causal)
    wq, wk, wv = reference_grads(q, k, v, dout, causal)
    check(dq, wq, f"dq {case} {dtype}")
    check(dk, wk, f"dk {case} {dtype}")
    check(dv, wv, f"dv {case} {dtype}")


def test_autograd_wrapper_on_the_device():
    g = torch.Generator().manual_seed(43)
    q = torch.randn(2, 4, 192, 128, generator=g).bfloat16()
    k = torch.randn(2, 2, 192, 128, generator=g).bfloat16()
    v = torch.randn(2, 2, 192, 128, generator=g).bfloat16()
    dout = torch.randn(2, 4, 192, 128, generator=g).bfloat16()
    dq_, dk_, dv_ = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = paras_nn.scaled_dot_product_attention(dq_, dk_, dv_, is_causal=True)
    out.backward(dout.to(DEV))
    wq, wk, wv = reference_grads(q, k, v, dout, True)
    check(dq_.grad, wq, "autograd dq")
    check(dk_.grad, wk, "autograd dk")
    check(dv_.grad, wv, "autograd dv")
    assert dk_.grad.shape == k.shape and dq_.grad.dtype == torch.bfloat16


def test_unsupported_operands_raise():
    q = torch.randn(1, 2, 64, 128, device=CUDA)
    with pytest.raises(RuntimeError):
        abi.sdpa_bwd(q, q, q, q, q, torch.zeros(1, 2, 64, device=CUDA))           # fp32
    h = torch.randn(1, 2, 60, 128, device=CUDA).bfloat16()
    with pytest.raises(RuntimeError):
        abi.sdpa_bwd(h, h, h, h, h, torch.zeros(1, 2, 60, device=CUDA))           # key length not a multiple of 8


def test_functional_ops_with_requires_grad_give_gradients_not_silence():
    # F.scaled_dot_product_attention / F.rms_norm / F.linear on `paras` tensors that require grad:
    # the reference differentiates through its composites, so the same Python calls must train here.
    g = torch.Generator().manual_seed(47)
    q = torch.randn(1, 4, 256, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 256, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 256, 128, generator=g).bfloat16()
    dout = torch.randn(1, 4, 256, 128, generator=g).bfloat16()
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=True)
    assert out.grad_fn is not None
    out.backward(dout.to(DEV))
    wq, wk, wv = reference_grads(q, k, v, dout, True)
    check(qd.grad, wq, "F.sdpa dq")
    check(kd.grad, wk, "F.sdpa dk")
    check(vd.grad, wv, "F.sdpa dv")
    # without grad the same call is the plain fused forward, and gives the same values
    with torch.no_grad():
        plain = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=True)
    assert plain.grad_fn is None and torch.equal(plain.cpu(), out.detach().cpu())
    # what the gradient does not cover raises instead of returning a result without grad_fn
    with pytest.raises(RuntimeError, match="gradient of the fused attention"):
        F.scaled_dot_product_attention(qd.float(), kd.float().repeat_interleave(2, 1),
                                       vd.float().repeat_interleave(2, 1))
    with pytest.raises(RuntimeError, match="gradient of the fused attention"):
        F.scaled_dot_product_attention(qd, qd, qd, attn_mask=torch.ones(256, 256, dtype=torch.bool).to(DEV))

    # rms_norm: fp32 (the reference's own test dtype) against CPU autograd
    x = torch.randn(6, 5, 32, generator=g)
    w = torch.randn(32, generator=g)
    xr, wr = x.clone().requires_grad_(), w.clone().requires_grad_()
    F.rms_norm(xr, (32,), wr, 1e-6).sum().backward()
    xd, wd = x.to(DEV).requires_grad_(), w.to(DEV).requires_grad_()
    y = F.rms_norm(xd, (32,), wd, 1e-6)
    assert y.grad_fn is not None and y.shape == x.shape
    y.sum().backward()
    assert torch.allclose(xd.grad.cpu(), xr.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(wd.grad.cpu(), wr.grad, atol=1e-4, rtol=1e-4)
    x2 = x.clone().requires_grad_()
    F.rms_norm(x2, (5, 32)).sum().backward()          # two trailing dims, no weight
    x2d = x.to(DEV).requires_grad_()
    F.rms_norm(x2d, (5, 32)).sum().backward()
    assert torch.allclose(x2d.grad.cpu(), x2.grad, atol=1e-4, rtol=1e-4)

    # linear: bf16 on the tensor-core GEMM, gradients by mm on the device
    a = torch.randn(3, 64, 256, generator=g).bfloat16()
    wl = (torch.randn(128, 256, generator=g) * 0.05).bfloat16()
    bl = torch.randn(128, generator=g).bfloat16()
    ar, wlr, blr = (t.double().requires_grad_() for t in (a, wl, bl))
    F.linear(ar, wlr, blr).sum().backward()
    ad, wld, bld = (t.to(DEV).requires_grad_() for t in (a, wl, bl))
    yl = F.linear(ad, wld, bld)
    assert yl.grad_fn is not None and yl.shape == (3, 64, 128)
    yl.sum().backward()
    for got, want, name in ((ad.grad, ar.grad, "dx"), (wld.grad, wlr.grad, "dw"), (bld.grad, blr.grad, "db")):
        err = (got.cpu().double() - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), f"linear {name}: {err}"
