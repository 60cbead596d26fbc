"""Rotary embedding: the stand-alone kernel, and attention with the rotation in its prologue
(paras_b200_sdpa_rope_fwd / paras::sdpa_rope), against the composition a user of the reference builds
from its operators: x * cos + rotate_half(x) * sin (paras::rotate_half, csrc/ops/fused_ops.cpp:234-267;
mul and add round to the tensor dtype, pointwise_ops.cpp:62-85) in front of sdpa_math
(attention_ops.cpp:71-136).  The rotation itself must be bit-exact; the attention behind it is held
to the usual tolerance (fp32 1e-4, 16 bit 2e-2)."""
import pytest
import torch

from oracle import oracle as O
from oracle import stats

import torch_paras  # noqa: F401
from torch_paras import abi, nn as paras_nn

pytestmark = pytest.mark.gpu
CUDA = "cuda:0"
DEV = "paras:1"


def tables(rows, D, dtype, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.arange(rows, dtype=torch.float64)[:, None] * inv[None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype)  # noqa: E731
    return mk(B, Hq, Lq, D), mk(B, Hkv, Lk, D), mk(B, Hkv, Lk, D)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 3, 50, 128), (1, 2, 300, 64), (1, 1, 7, 6)])
def test_rope_kernel_is_bit_exact(shape, dtype):
    B, H, L, D = shape
    x, _, _ = qkv(B, H, H, L, L, D, dtype, 3)
    cos, sin = tables(L + 5, D, dtype)
    got = abi.rope(x.to(CUDA), cos.to(CUDA), sin.to(CUDA), pos0=5)
    assert torch.equal(got.cpu(), O.rope(x, cos, sin, 5))
    xt = x.transpose(1, 2).contiguous().transpose(1, 2)          # [B, L, H, D] storage
    assert torch.equal(abi.rope(xt.to(CUDA).transpose(1, 2).contiguous().transpose(1, 2), cos.to(CUDA), sin.to(CUDA), pos0=5).cpu(),
                       O.rope(x, cos, sin, 5))


CASES = [
    # B, Hq, Hkv, Lq, Lk, D, causal
    (1, 2, 2, 256, 256, 128, True),
    (2, 8, 2, 640, 640, 128, True),      # GQA, odd number of query tiles
    (1, 4, 1, 300, 300, 128, True),      # ragged rows: the last tile is partly past the end
    (1, 2, 2, 200, 456, 128, False),     # Lq != Lk
    (1, 4, 4, 333, 333, 64, True),       # head dim 64: queries rotated by the streaming pass
    (2, 8, 2, 1, 700, 128, False),       # decode step: one query at position 699
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("case", CASES)
def test_attention_with_rope_prologue(case, dtype):
    B, Hq, Hkv, Lq, Lk, D, causal = case
    q, k, v = qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=Lq + Lk)
    q_pos0 = Lk - Lq if Lq == 1 else 0
    cos, sin = tables(max(Lq + q_pos0, Lk), D, dtype)
    want = O.sdpa(O.rope(q, cos, sin, q_pos0), O.rope(k, cos, sin, 0), v, is_causal=causal, enable_gqa=Hq != Hkv)
    got = abi.sdpa_rope_fwd(q.to(CUDA), k.to(CUDA), v.to(CUDA), cos.to(CUDA), sin.to(CUDA), causal=causal,
                            q_pos0=q_pos0, flags=abi.SDPA_REF_SCALE)
    if dtype != torch.float32 and D == 128 and Lq > 16:
        assert abi.sdpa_last_kernel() == "tcgen05_rope"           # the in-kernel rotation really ran
    if dtype == torch.float32:
        assert torch.allclose(got.cpu(), want, atol=1e-4, rtol=1e-4)
    else:
        r = stats.report(got, want, 2e-2)
        print(f"rope + sdpa {case} {dtype}: {stats.fmt(r)}")
        assert r["over_tol"] == 0 and r["max_abs"] <= 2e-2, stats.fmt(r)
    # the same through the operator on the device
    out = paras_nn.attention_rope(q.to(DEV), k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV), is_causal=causal,
                                  q_pos0=q_pos0)
    assert torch.equal(out.cpu(), got.cpu())
    assert torch.equal(paras_nn.rope(k.to(DEV), cos.to(DEV), sin.to(DEV)).cpu(), O.rope(k, cos, sin))


def test_rope_argument_errors():
    q, k, v = qkv(1, 2, 2, 64, 64, 128, torch.bfloat16, 1)
    cos, sin = tables(32, 128, torch.bfloat16)                       # too few positions
    with pytest.raises(RuntimeError, match="positions"):
        paras_nn.attention_rope(q.to(DEV), k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV))
    with pytest.raises(RuntimeError, match="do not cover"):
        abi.sdpa_rope_fwd(q.to(CUDA), k.to(CUDA), v.to(CUDA), cos.to(CUDA), sin.to(CUDA))
