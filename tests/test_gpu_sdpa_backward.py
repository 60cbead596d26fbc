"""Attention backward (paras_b200_sdpa_bwd, torch_paras.nn.scaled_dot_product_attention).

Two expectations.  (1) The reference's own gradients: autograd through its composite attention
(csrc/ops/attention_ops.cpp:71-136, softmax backward pointwise_ops.cpp:994-1062) on its paras:0
engine, committed as fixtures tests/golden/sdpa_grad_*.pt.  The reference can only differentiate
3-D (batch, seq, dim) inputs -- with 4-D inputs its backward of the batched product raises -- so
those fixtures have one head per batch entry.  (2) The gradient of float64 attention on the same
16-bit inputs, for everything the fixtures cannot cover (GQA sums, many tiles, ragged shapes).

The reference rounds scores, probabilities and their gradients to 16 bits; its own gradients
differ from the float64 ones by up to 1 % of a gradient's largest entry (0.05 % on average).  The
kernels keep S, P and dP in fp32 and round P and dS once.  Bound, per element:
    |got - want| <= 2 ulp(|want|) + 8e-3 * max|want|      and a mean error below 1e-3 * max|want|.
"""
import math

import pytest
import torch
import torch.nn.functional as F

from conftest import golden_names, load_golden
from oracle import stats

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


def check(got, want, name, c=8e-3, mean_c=1e-3):
    dtype = got.dtype
    got = got.detach().cpu().double()
    want = want.double()
    scale = want.abs().max().item()
    err = (got - want).abs()
    assert torch.isfinite(got).all(), name
    bound = 2 * stats.ulp_of(want.to(dtype)) + c * scale
    worst = (err - bound).max().item()
    print(f"{name}: max error {err.max().item():.3e} ({err.max().item() / scale:.2e} of scale), "
          f"mean {err.mean().item() / scale:.2e} of scale")
    assert worst <= 0, f"{name}: an element exceeds 2 ulp + {c} * scale by {worst:.3e} (scale {scale:.3e})"
    assert err.mean().item() <= mean_c * scale, f"{name}: mean error {err.mean().item():.3e} vs scale {scale:.3e}"


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


@pytest.mark.parametrize("path", ["fused", "composite"])
@pytest.mark.parametrize("name", golden_names("sdpa_grad"))
def test_backward_against_the_reference_gradients(name, path):
    g = load_golden(name)
    a = g["args"]
    _, wq, wk, wv = g["out"]
    # (batch, seq, dim) -> [batch, 1 head, seq, dim]
    q, k, v, dout = (a[n].unsqueeze(1).to(CUDA) for n in ("q", "k", "v", "dout"))
    causal = bool(a.get("is_causal", False))
    out, lse = abi.sdpa_fwd(q, k, v, causal=causal, return_lse=True, flags=abi.SDPA_REF_SCALE)
    sc = float(torch.tensor(1 / math.sqrt(q.shape[-1])).to(q.dtype))     # the scale the forward used
    dq, dk, dv = abi.sdpa_bwd(dout, q, k, v, out, lse, causal=causal, scale=sc, composite=path == "composite")
    # against gradients that carry the reference's own 16-bit rounding noise (up to 1 % of scale)
    check(dq.squeeze(1), wq, f"{name} dq [{path}]", c=1.5e-2, mean_c=2e-3)
    check(dk.squeeze(1), wk, f"{name} dk [{path}]", c=1.5e-2, mean_c=2e-3)
    check(dv.squeeze(1), wv, f"{name} dv [{path}]", c=1.5e-2, mean_c=2e-3)


CASES += [
    (1, 8, 2, 2048, 2048, 128, True),    # 16 x 16 tiles per head, GQA 4:1: long accumulation chains
    (2, 2, 2, 520, 130, 128, True),      # key tiles that only the last query tiles see; ragged both ways
    (1, 2, 1, 130, 520, 128, True),      # more keys than queries: key tiles no query sees get zeros
    (1, 3, 3, 77, 77, 64, False),        # a single ragged tile
]


@pytest.mark.parametrize("path", ["fused", "composite"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_backward_through_the_c_abi(case, dtype, path):
    B, Hq, Hkv, Lq, Lk, D, causal = case
    if path == "composite" and Lk % 8:
        pytest.skip("the composite path needs a key length that is a multiple of 8")
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
    dq, dk, dv = abi.sdpa_bwd(dd, qd, kd, vd, out, lse, causal=causal, composite=path == "composite")
    wq, wk, wv = reference_grads(q, k, v, dout, causal)
    # the composite path rounds the four [L, L] matrices to 16 bits like the reference: looser
    c, mc = (8e-3, 1e-3) if path == "fused" else (3e-2, 1e-2)
    check(dq, wq, f"dq {case} {dtype} [{path}]", c, mc)
    check(dk, wk, f"dk {case} {dtype} [{path}]", c, mc)
    check(dv, wv, f"dv {case} {dtype} [{path}]", c, mc)


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


@pytest.mark.parametrize("kind", ["bool", "additive", "additive_4d_min"])
def test_a_causal_mask_passed_as_a_tensor_trains_through_the_fused_kernels(kind):
    # F.scaled_dot_product_attention(q, k, v, attn_mask=<the lower triangle>) with requires_grad: the operator
    # layer asks the GPU whether the mask is the causal mask and, if so, runs the call as is_causal=True:
    # output and gradients equal that call's bit for bit.  A mask one entry off takes the general route
    # and still matches float64.
    g = torch.Generator().manual_seed(53)
    q = torch.randn(2, 4, 320, 128, generator=g).bfloat16()
    k = torch.randn(2, 2, 320, 128, generator=g).bfloat16()
    v = torch.randn(2, 2, 320, 128, generator=g).bfloat16()
    dout = torch.randn(2, 4, 320, 128, generator=g).bfloat16()
    tri = torch.ones(320, 320, dtype=torch.bool).tril()

    def as_kind(t):
        if kind == "bool":
            return t
        if kind == "additive":
            return torch.zeros(320, 320).masked_fill(~t, float("-inf")).bfloat16()
        return torch.zeros(1, 1, 320, 320, dtype=torch.bfloat16).masked_fill(~t, torch.finfo(torch.bfloat16).min)

    def run(**kw):
        qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
        out = F.scaled_dot_product_attention(qd, kd, vd, enable_gqa=True, **kw)
        out.backward(dout.to(DEV))
        return out.detach().cpu(), qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu()

    ref = run(is_causal=True)
    mask_dev = as_kind(tri).to(DEV)
    for _ in range(2):                       # the second call answers from the remembered check
        got = run(attn_mask=mask_dev)
        for a_, b_ in zip(got, ref):
            assert torch.equal(a_, b_)
    off = tri.clone()
    off[200, 250] = True
    got = run(attn_mask=as_kind(off).to(DEV))
    assert not torch.equal(got[0], ref[0])
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    s_ = (q64 @ k64.repeat_interleave(2, 1).transpose(-1, -2)) / math.sqrt(128)
    want = torch.softmax(s_.masked_fill(~off, float("-inf")), -1) @ v64.repeat_interleave(2, 1)
    want.backward(dout.double())
    assert (got[0].double() - want.detach()).abs().max().item() <= 2e-2
    for got_g, want_g in zip(got[1:], (q64.grad, k64.grad, v64.grad)):
        assert (got_g.double() - want_g).abs().max().item() <= 2e-2 * max(want_g.abs().max().item(), 1e-2)
    # the remembered answer follows the tensor, not the address: writing into the mask, or a new mask of the same
    # shape (which the allocator may place where an old one was), is looked at again
    m2 = as_kind(tri).to(DEV)
    assert torch.equal(run(attn_mask=m2)[0], ref[0])
    if kind == "bool":
        m2[200, 250] = True
    else:
        m2[..., 200, 250] = 0
    assert not torch.equal(run(attn_mask=m2)[0], ref[0])
    del m2
    m3 = as_kind(off).to(DEV)
    assert not torch.equal(run(attn_mask=m3)[0], ref[0])
    # the check itself, through the C ABI
    assert abi.sdpa_mask_is_causal(tri.to(CUDA), torch.bfloat16) and not abi.sdpa_mask_is_causal(off.to(CUDA), torch.bfloat16)


def test_unsupported_operands_raise():
    q = torch.randn(1, 2, 64, 128, device=CUDA)
    with pytest.raises(RuntimeError):
        abi.sdpa_bwd(q, q, q, q, q, torch.zeros(1, 2, 64, device=CUDA))           # fp32
    h = torch.randn(1, 2, 60, 128, device=CUDA).bfloat16()
    with pytest.raises(RuntimeError):
        abi.sdpa_bwd(h, h, h, h, h, torch.zeros(1, 2, 60, device=CUDA), composite=True)   # key length not a multiple of 8


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
    # what the fused kernels do not take (fp32, a mask tensor, dropout, 3-D inputs) goes to the general
    # backward, never to a result without grad_fn: checked against CPU autograd on the same inputs
    g2 = torch.Generator().manual_seed(48)
    q3, k3, v3, d3 = (torch.randn(3, 50, 32, generator=g2) for _ in range(4))          # 3-D fp32, as the reference's tests
    pad = torch.ones(3, 50, 50, dtype=torch.bool)
    pad[:, :, 40:] = False                                                                # per-batch key padding
    cq, ck, cv = (t.clone().requires_grad_(True) for t in (q3, k3, v3))
    F.scaled_dot_product_attention(cq, ck, cv, attn_mask=pad).backward(d3)
    dq3, dk3, dv3 = (t.to(DEV).requires_grad_(True) for t in (q3, k3, v3))
    o3 = F.scaled_dot_product_attention(dq3, dk3, dv3, attn_mask=pad.to(DEV))
    assert o3.grad_fn is not None
    o3.backward(d3.to(DEV))
    for got, want, name in ((dq3.grad, cq.grad, "dq"), (dk3.grad, ck.grad, "dk"), (dv3.grad, cv.grad, "dv")):
        assert got.shape == want.shape
        assert torch.allclose(got.cpu(), want, atol=1e-4, rtol=1e-4), f"masked fp32 3-D {name}"
    # dropout: the backward replays the forward's draw -- dv = wd^T dO is linear in dO with the same weights
    torch_paras.manual_seed(5)
    qh, kh, vh = (torch.randn(1, 2, 64, 64, generator=g2).bfloat16().to(DEV).requires_grad_(True) for _ in range(3))
    od = F.scaled_dot_product_attention(qh, kh, vh, dropout_p=0.5)
    assert od.grad_fn is not None
    od.backward(torch.ones_like(od))
    assert torch.isfinite(qh.grad.float()).all() and vh.grad.float().abs().sum().item() > 0
    # column sums of the dropped weights: dv[j, :] = sum_i wd[i, j] for dO = 1; the forward's output row sums
    # give sum_j wd[i, j] v[j, :]; both come from the same wd, so sum_j dv[j, 0] * 1 == sum_i rowsum(wd[i])
    with torch.no_grad():
        torch_paras.manual_seed(5)
        ones_v = torch.ones_like(vh)
        rows = F.scaled_dot_product_attention(qh, kh, ones_v, dropout_p=0.5)              # = rowsum(wd), same draw
    assert abs(vh.grad[..., 0].float().sum().item() - rows[..., 0].float().sum().item()) <= 0.02 * rows[..., 0].numel()

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


def test_fused_backward_is_deterministic_and_leaves_inputs_alone():
    # no atomics and one owner per accumulator: two runs give the same bits, with other work in between
    g = torch.Generator().manual_seed(77)
    B, Hq, Hkv, L, D = 2, 8, 2, 700, 128
    q, k, v, do = (torch.randn(B, h, L, D, generator=g).bfloat16().to(CUDA) for h in (Hq, Hkv, Hkv, Hq))
    o, lse = abi.sdpa_fwd(q, k, v, causal=True, return_lse=True)
    keep = [t.clone() for t in (q, k, v, do, o, lse)]
    first = abi.sdpa_bwd(do, q, k, v, o, lse, causal=True)
    abi.sdpa_fwd(k, k, v, causal=False)                       # other kernels reuse TMEM and the pool's scratch
    abi.sdpa_bwd(do.flip(0), q, k, v, o, lse, causal=True)
    second = abi.sdpa_bwd(do, q, k, v, o, lse, causal=True)
    for a, b, name in zip(first, second, ("dq", "dk", "dv")):
        assert torch.equal(a, b), f"{name} differs between two runs"
    for a, b in zip(keep, (q, k, v, do, o, lse)):
        assert torch.equal(a, b)


def _float64_grads(q, k, v, dout, *, causal=False, mask=None, keep=None):
    """Gradients of float64 attention on the same inputs; `keep` multiplies the weights (dropout)."""
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    r = q.shape[1] // k.shape[1]
    kk, vv = k64.repeat_interleave(r, 1), v64.repeat_interleave(r, 1)
    s = (q64 @ kk.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if causal:
        s = s.masked_fill(~torch.ones(q.shape[2], k.shape[2], dtype=torch.bool).tril(), float("-inf"))
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else s + mask.double()
    w = torch.softmax(s, -1)
    if keep is not None:
        w = w * keep.double()
    (w @ vv).backward(dout.double())
    return q64.grad, k64.grad, v64.grad


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["bool_mask", "additive_mask", "causal_odd_dim", "dropout_mask", "philox"])
def test_general_backward_covers_masks_dropout_and_fp32(kind, dtype):
    # the cases the fused kernels do not take, on the CUDA-core path (paras_b200_sdpa_bwd_general)
    g = torch.Generator().manual_seed(91)
    B, Hq, Hkv, Lq, Lk, D = 2, 4, 2, 70, 90, 40 if kind == "causal_odd_dim" else 64
    q, k, v, do = (torch.randn(B, h, L, D, generator=g).to(dtype) for h, L in ((Hq, Lq), (Hkv, Lk), (Hkv, Lk), (Hq, Lq)))
    kw, ref_kw = {}, {}
    if kind == "bool_mask":
        m = torch.rand(B, 1, Lq, Lk, generator=g) > 0.3
        m[..., 0] = True
        kw["mask"], ref_kw["mask"] = m.to(CUDA), m
    elif kind == "additive_mask":
        m = torch.randn(Lq, Lk, generator=g).to(dtype)
        kw["mask"], ref_kw["mask"] = m.to(CUDA), m
    elif kind == "causal_odd_dim":
        kw["causal"] = ref_kw["causal"] = True
    elif kind == "dropout_mask":
        dm = (torch.rand(B, Hq, Lq, Lk, generator=g) > 0.4).to(dtype)
        kw.update(dropout_p=0.25, dropout_mask=dm.to(CUDA))
        one_minus_p = float(torch.tensor(0.75).to(dtype))
        ref_kw["keep"] = dm.double() / one_minus_p
    else:
        # the forward's Philox draws, rebuilt on the host by the oracle (random_ops.cpp:27-47, 140-176)
        from oracle import oracle as O
        kw.update(dropout_p=0.2, rng=(1234, 7))
        import numpy as np
        r0 = O.philox2x32_r0(1234, 7, B * Hq * Lq * Lk)
        u = (r0 >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)
        keep = torch.from_numpy(u < np.float32(1.0 - 0.2)).reshape(B, Hq, Lq, Lk)
        ref_kw["keep"] = keep.double() * float(np.float32(1.0) / np.float32(1.0 - 0.2))
    got = abi.sdpa_bwd_general(do.to(CUDA), q.to(CUDA), k.to(CUDA), v.to(CUDA), **kw)
    want = _float64_grads(q, k, v, do, **ref_kw)
    c = 1e-4 if dtype == torch.float32 else 8e-3
    for a, b, name in zip(got, want, ("dq", "dk", "dv")):
        check(a, b, f"general {kind} {dtype} {name}", c=c, mean_c=c / 8)
