"""Pins the CPU oracle (oracle/oracle.py) against
  (a) the committed golden vectors, which are outputs of the unmodified reference build
      on its paras:0 host engine (tests/golden/make_golden.py), bit for bit;
  (b) what the reference's own tests assert for this path: agreement with CPU PyTorch at
      atol = rtol = 1e-4 on their fp32 shapes (tests/test_attention_norm_ops.py:35-165,
      tests/test_fused_ops.py:12-70 of the reference);
  (c) the live reference build, when oracle/_ref/_C.so is present.
"""
import math
import os
import subprocess
import sys
import tempfile

import pytest
import torch
import torch.nn.functional as F

from conftest import ROOT, golden_names, load_golden
from oracle import oracle as O


def run_oracle(op, a):
    if op == "sdpa":
        return O.sdpa(a["q"], a["k"], a["v"], attn_mask=a.get("attn_mask"),
                      is_causal=bool(a.get("is_causal", False)), scale=a.get("scale"),
                      enable_gqa=bool(a.get("enable_gqa", False)))
    if op == "sdpa_math":   # (output, weights after dropout); the reference was re-seeded: sequence 0
        return O.sdpa(a["q"], a["k"], a["v"], attn_mask=a.get("attn_mask"),
                      is_causal=bool(a.get("is_causal", False)), scale=a.get("scale"),
                      enable_gqa=bool(a.get("enable_gqa", False)), return_weights=True,
                      dropout_p=float(a.get("dropout_p", 0.0)), dropout_mask=a.get("dropout_mask"),
                      rng=(int(a.get("seed", 0)), 0))
    if op == "rms_norm_aten":
        return O.rms_norm_composite(a["x"], a["normalized_shape"], a.get("weight"), a.get("eps"))
    if op == "rms_norm_paras":
        return O.rms_norm_fused(a["x"], a["weight"], a["eps"])
    if op == "rms_norm_paras_backward":
        return O.rms_norm_fused_backward(a["grad_out"], a["x"], a["weight"], a["rstd"])
    if op == "swiglu_paras":
        return O.swiglu_fused(a["gate"], a["up"])
    if op == "swiglu_paras_backward":
        return O.swiglu_fused_backward(a["grad_out"], a["gate"], a["up"])
    if op == "swiglu_composite":
        return O.swiglu_composite(a["x"], a["gate"])
    if op == "rotate_half":
        return O.rotate_half(a["x"])
    if op == "rotate_half_backward":
        return O.rotate_half_backward(a["grad_out"])
    if op == "rope_sdpa":   # (rotated q, rotated k, attention over them)
        qr = O.rope(a["q"], a["cos"], a["sin"], int(a.get("q_pos0", 0)))
        kr = O.rope(a["k"], a["cos"], a["sin"], 0)
        return qr, kr, O.sdpa(qr, kr, a["v"], is_causal=bool(a.get("is_causal", False)),
                              enable_gqa=bool(a.get("enable_gqa", False)))
    raise AssertionError(op)


def as_tuple(x):
    return x if isinstance(x, tuple) else (x,)


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_golden_bit_exact(name):
    g = load_golden(name)
    got = as_tuple(run_oracle(g["op"], g["args"]))
    want = as_tuple(g["out"])
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert a.dtype == b.dtype and a.shape == b.shape
        assert torch.equal(a, b) or torch.allclose(a.double(), b.double(), rtol=0, atol=0, equal_nan=True), \
            f"{name}: max-abs {(a.double() - b.double()).abs().max().item()}"


def _close(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    assert torch.allclose(a, b, atol=1e-4, rtol=1e-4, equal_nan=True)


def _qkv(B=2, H=4, Lq=8, Lk=8, E=16):
    return torch.randn(B, H, Lq, E), torch.randn(B, H, Lk, E), torch.randn(B, H, Lk, E)


def test_reference_test_expectations_sdpa():
    torch.manual_seed(0)
    q, k, v = _qkv()
    _close(O.sdpa(q, k, v), F.scaled_dot_product_attention(q, k, v))
    s = 1.0 / math.sqrt(32)
    _close(O.sdpa(q, k, v, scale=s), F.scaled_dot_product_attention(q, k, v, scale=s))
    _close(O.sdpa(q, k, v, is_causal=True), F.scaled_dot_product_attention(q, k, v, is_causal=True))
    q2, k2, v2 = _qkv(Lq=4, Lk=8)  # top-left aligned causal mask
    _close(O.sdpa(q2, k2, v2, is_causal=True),
           F.scaled_dot_product_attention(q2, k2, v2, is_causal=True))
    mask = torch.rand(2, 4, 8, 8) > 0.3
    _close(O.sdpa(q, k, v, attn_mask=mask), F.scaled_dot_product_attention(q, k, v, attn_mask=mask))
    bias = torch.randn(2, 4, 8, 8) * 0.1
    _close(O.sdpa(q, k, v, attn_mask=bias), F.scaled_dot_product_attention(q, k, v, attn_mask=bias))
    qg, kg, vg = torch.randn(2, 4, 8, 16), torch.randn(2, 2, 8, 16), torch.randn(2, 2, 8, 16)
    ref, _ = torch.ops.aten._scaled_dot_product_attention_math(
        qg, kg, vg, None, 0.0, False, None, scale=None, enable_gqa=True)
    _close(O.sdpa(qg, kg, vg, enable_gqa=True), ref)
    with pytest.raises(RuntimeError):
        O.sdpa(torch.randn(1, 5, 4, 8), torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8), enable_gqa=True)


def test_reference_test_expectations_norm_glu():
    torch.manual_seed(0)
    x = torch.randn(4, 6, 32)
    w = torch.randn(32)
    _close(O.rms_norm_composite(x, [32], None, None), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6))
    _close(O.rms_norm_composite(x, [32], w, 1e-5), torch.ops.aten.rms_norm(x, [32], w, 1e-5))
    x3 = torch.randn(3, 4, 5)
    _close(O.rms_norm_composite(x3, [4, 5], None, 1e-6), torch.ops.aten.rms_norm(x3, [4, 5], None, 1e-6))
    with pytest.raises(RuntimeError):
        O.rms_norm_composite(x, [32], torch.randn(16), None)
    x2, w2 = torch.randn(4, 8), torch.randn(8)
    _close(O.rms_norm_fused(x2, w2, 1e-6)[0], x2 * torch.rsqrt(x2.pow(2).mean(-1, keepdim=True) + 1e-6) * w2)
    gate, up = torch.randn(4, 8), torch.randn(4, 8)
    _close(O.swiglu_fused(gate, up), F.silu(gate) * up)
    _close(O.swiglu_composite(up, gate), up * F.silu(gate))
    x1, x2h = x2.chunk(2, dim=-1)
    _close(O.rotate_half(x2), torch.cat((-x2h, x1), dim=-1))
    # backward formulas against autograd
    xg, wg = x2.clone().requires_grad_(), w2.clone().requires_grad_()
    (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + 1e-6) * wg).sum().backward()
    _, rstd = O.rms_norm_fused(x2, w2, 1e-6)
    gi, gw = O.rms_norm_fused_backward(torch.ones(4, 8), x2, w2, rstd)
    _close(gi, xg.grad)
    _close(gw, wg.grad)
    gg, ug = gate.clone().requires_grad_(), up.clone().requires_grad_()
    (F.silu(gg) * ug).sum().backward()
    dg, du = O.swiglu_fused_backward(torch.ones(4, 8), gate, up)
    _close(dg, gg.grad)
    _close(du, ug.grad)


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "_C.so")),
                    reason="reference build (oracle/_ref) not present")
def test_oracle_matches_live_reference_bf16_seeded():
    g = torch.Generator().manual_seed(99)
    q = torch.randn(1, 4, 96, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 96, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 96, 128, generator=g).bfloat16()
    x = torch.randn(32, 512, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(512, generator=g)).bfloat16()
    jobs = [{"op": "sdpa", "args": {"q": q, "k": k, "v": v, "is_causal": True, "enable_gqa": True}},
            {"op": "rms_norm_aten", "args": {"x": x, "weight": w, "normalized_shape": [512], "eps": 1e-6}},
            {"op": "swiglu_paras", "args": {"gate": x, "up": x.flip(0)}}]
    want = [O.sdpa(q, k, v, is_causal=True, enable_gqa=True), O.rms_norm_composite(x, [512], w, 1e-6),
            O.swiglu_fused(x, x.flip(0))]
    with tempfile.TemporaryDirectory() as td:
        torch.save(jobs, os.path.join(td, "j.pt"))
        subprocess.check_call([sys.executable, os.path.join(ROOT, "oracle", "ref_run.py"),
                               os.path.join(td, "j.pt"), os.path.join(td, "r.pt")])
        res = torch.load(os.path.join(td, "r.pt"))
    for r, w_ in zip(res, want):
        assert torch.equal(r["out"], w_)
