"""Pins the plain-C restatement (oracle/paras_oracle.c) against the golden vectors of the
unmodified reference and against the torch restatement (oracle/oracle.py).

Bit-exact wherever the reference's own arithmetic is written out (RMSNorm both ways, SwiGLU
both ways, their backward ops, rotate_half, softmax).  For attention the reference's two
matrix products run in libtorch's blocked CPU kernels, whose summation order the C code
does not restate; there the bound is one rounding step of the storage type.
"""
import numpy as np
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import c_oracle as C
from oracle import oracle as O


def run_c(op, a):
    if op == "sdpa":
        return C.sdpa(a["q"], a["k"], a["v"], attn_mask=a.get("attn_mask"),
                      is_causal=bool(a.get("is_causal", False)), scale=a.get("scale"),
                      enable_gqa=bool(a.get("enable_gqa", False)))
    if op == "rms_norm_aten":
        return C.rms_norm_composite(a["x"], a["normalized_shape"], a.get("weight"), a.get("eps"))
    if op == "rms_norm_paras":
        return C.rms_norm_fused(a["x"], a["weight"], a["eps"])
    if op == "rms_norm_paras_backward":
        return C.rms_norm_fused_backward(a["grad_out"], a["x"], a["weight"], a["rstd"])
    if op == "swiglu_paras":
        return C.swiglu_fused(a["gate"], a["up"])
    if op == "swiglu_paras_backward":
        return C.swiglu_fused_backward(a["grad_out"], a["gate"], a["up"])
    if op == "swiglu_composite":
        return C.swiglu_composite(a["x"], a["gate"])
    if op == "rotate_half":
        return C.rotate_half(a["x"])
    if op == "rotate_half_backward":
        return C.rotate_half_backward(a["grad_out"])
    raise AssertionError(op)


def as_tuple(x):
    return x if isinstance(x, tuple) else (x,)


def same_bits(a, b):
    return a.dtype == b.dtype and a.shape == b.shape and \
        torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


# the C restatement has no dropout / weights output and no rotary composition: those fixtures pin the
# torch restatement only
@pytest.mark.parametrize("name", [n for n in golden_names() if not n.startswith(("sdpa_math", "rope_"))])
def test_c_oracle_matches_reference_golden(name):
    g = load_golden(name)
    got = as_tuple(run_c(g["op"], g["args"]))
    want = as_tuple(g["out"])
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert a.dtype == b.dtype and a.shape == b.shape
        if g["op"] == "sdpa":
            # outputs are averages of N(0,1) values: magnitude below 4, so one rounding step of the
            # storage type is 2^-22 (fp32) or 2^-7 (bf16)
            tol = 2.0 ** -7 if a.dtype == torch.bfloat16 else 2e-6
            err = (a.double() - b.double()).abs().max().item()
            assert err <= tol, f"{name}: max-abs {err}"
        else:
            assert same_bits(a, b), f"{name}: max-abs {(a.double() - b.double()).abs().max().item()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_c_oracle_matches_torch_restatement(dtype):
    g = torch.Generator().manual_seed(7)
    x = (3.0 * torch.randn(19, 130, generator=g)).to(dtype)
    w = (1 + 0.2 * torch.randn(130, generator=g)).to(dtype)
    y = torch.randn(19, 130, generator=g).to(dtype)
    for a, b in zip(C.rms_norm_fused(x, w, 1e-5), O.rms_norm_fused(x, w, 1e-5)):
        assert same_bits(a, b)
    assert same_bits(C.rms_norm_composite(x, [130], w, 1e-5), O.rms_norm_composite(x, [130], w, 1e-5))
    assert same_bits(C.rms_norm_composite(x, [130], None, None), O.rms_norm_composite(x, [130], None, None))
    assert same_bits(C.swiglu_fused(x, y), O.swiglu_fused(x, y))
    assert same_bits(C.swiglu_composite(y, x), O.swiglu_composite(y, x))
    for a, b in zip(C.swiglu_fused_backward(y, x, w.expand_as(x)), O.swiglu_fused_backward(y, x, w.expand_as(x))):
        assert same_bits(a, b)
    rstd = O.rms_norm_fused(x, w, 1e-5)[1]
    for a, b in zip(C.rms_norm_fused_backward(y, x, w, rstd), O.rms_norm_fused_backward(y, x, w, rstd)):
        assert same_bits(a, b)
    assert same_bits(C.rotate_half(x), O.rotate_half(x))
    assert same_bits(C.rotate_half_backward(x), O.rotate_half_backward(x))
    with pytest.raises(RuntimeError):
        C.rotate_half(x[:, :129])
    s = (4.0 * torch.randn(11, 77, generator=g)).to(dtype)
    s[3, 5:] = float("-inf")
    a, b = C.softmax_lastdim(s), O.softmax_lastdim(s)
    # libm's exp and torch's vectorised exp may differ in the last bit of a double: after the
    # rounding to the storage type that shows, if ever, as one step
    assert (a.double() - b.double()).abs().max().item() <= (2.0 ** -8 if dtype != torch.float32 else 2.0 ** -23)


def test_c_oracle_conversions_exhaustive_16bit():
    """Every bf16 and fp16 bit pattern survives 16 -> 32 -> 16, and float -> 16-bit rounding agrees
    with torch's on a dense sample that includes ties, subnormals and the overflow edge."""
    lib = C.load()
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    for dt, to32, to16 in ((torch.bfloat16, lib.po_bf16_to_f32, lib.po_f32_to_bf16),
                           (torch.float16, lib.po_f16_to_f32, lib.po_f32_to_f16)):
        ref32 = bits.view(dt).float()
        for i in range(0, 65536, 7):
            h = int(bits[i].item()) & 0xFFFF
            f = to32(h)
            r = ref32[i].item()
            if np.isnan(r):
                assert np.isnan(f)
                continue
            assert f == r, (dt, hex(h))
            assert to16(f) == h, (dt, hex(h))
    g = torch.Generator().manual_seed(3)
    vals = torch.cat([torch.randn(4000, generator=g) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    ties = torch.tensor([1.00390625, 1.01171875, 65504.0, 65519.99, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8,
                         2.9802322387695312e-08, 8.940696716308594e-08, float("inf"), -0.0])
    vals = torch.cat([vals, ties, -ties])
    for dt, to16 in ((torch.bfloat16, lib.po_f32_to_bf16), (torch.float16, lib.po_f32_to_f16)):
        want = vals.to(dt).view(torch.int16)
        for i in range(vals.numel()):
            assert to16(vals[i].item()) == (int(want[i].item()) & 0xFFFF), (dt, vals[i].item())


def test_c_oracle_sdpa_tracks_torch_restatement_bf16():
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 4, 33, 64, generator=g).bfloat16()
    k = torch.randn(1, 2, 50, 64, generator=g).bfloat16()
    v = torch.randn(1, 2, 50, 64, generator=g).bfloat16()
    a = C.sdpa(q, k, v, is_causal=True, enable_gqa=True)
    b = O.sdpa(q, k, v, is_causal=True, enable_gqa=True)
    assert (a.double() - b.double()).abs().max().item() <= 2.0 ** -7
    with pytest.raises(RuntimeError):
        C.sdpa(torch.randn(1, 5, 4, 8), torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8), enable_gqa=True)
