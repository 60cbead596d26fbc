"""Seeded random shapes through every attention path (tcgen05, decode, CUDA-core; causal, bool / additive /
padding masks; fused, composite and general backward) against float64 attention on the same inputs.
The shapes mix tile multiples with ragged lengths, single rows and keys, GQA ratios and head dims from
32 to 256; forward tolerance 1e-4 (fp32) / 2e-2 (16 bit), gradients 2e-4 / 2e-2 of each gradient's
largest entry."""
import math
import random

import pytest
import torch

import torch_paras  # noqa: F401
from torch_paras import abi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def scores64(q, k, causal, mask):
    r = q.shape[1] // k.shape[1]
    s = (q @ k.repeat_interleave(r, 1).transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if causal:
        s = s.masked_fill(~torch.ones(q.shape[2], k.shape[2], dtype=torch.bool).tril(), float("-inf"))
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else s + mask.double()
    return s


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_shapes_forward_and_backward(seed):
    rnd = random.Random(seed)
    seen = set()
    for it in range(40):
        dtype = rnd.choice([torch.bfloat16, torch.float16, torch.float32])
        D = rnd.choice([128, 128, 128, 64, 64, 32, 40, 96, 256])
        Hkv = rnd.choice([1, 2, 3])
        Hq = Hkv * rnd.choice([1, 2, 4])
        B = rnd.choice([1, 2])
        Lq = rnd.choice([1, 2, 7, 64, 127, 128, 129, 200, 256, 300, 511, 640])
        Lk = rnd.choice([1, 5, 63, 64, 65, 128, 130, 255, 256, 257, 400, 700, 1000])
        causal = rnd.random() < 0.4
        kind = None if causal else rnd.choice([None, None, "bool", "add", "addf32", "pad", "tril", "trilpad"])
        g = torch.Generator().manual_seed(seed * 1000 + it)
        q = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
        k = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
        v = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
        do = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
        mask = None
        if kind == "bool":
            mask = torch.rand(B, Hq, Lq, Lk, generator=g) > 0.3
            mask[..., 0] = True
        elif kind == "add":
            mask = torch.randn(Lq, Lk, generator=g).to(dtype)
        elif kind == "addf32":
            mask = torch.randn(B, 1, Lq, Lk, generator=g)
        elif kind == "pad":
            mask = torch.ones(B, 1, 1, Lk, dtype=torch.bool)
            mask[:, :, :, Lk - Lk // 3:] = False
            mask[..., 0] = True
        elif kind == "tril":          # the causal mask written out, bool or additive
            tri = torch.ones(Lq, Lk, dtype=torch.bool).tril()
            mask = tri if rnd.random() < 0.5 else torch.zeros(Lq, Lk).masked_fill(~tri, float("-inf")).to(dtype)
        elif kind == "trilpad":       # causal over sequences padded on the right
            tri = torch.ones(Lq, Lk, dtype=torch.bool).tril()
            lens = [max(1, Lk - b * (Lk // 3)) for b in range(B)]
            mask = torch.stack([tri & (torch.arange(Lk)[None, :] < n) for n in lens])[:, None]
        tag = f"seed {seed} case {it}: {dtype} B{B} Hq{Hq} Hkv{Hkv} Lq{Lq} Lk{Lk} D{D} causal={causal} mask={kind}"
        dm = None if mask is None else mask.to(DEV)
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)

        got = abi.sdpa_fwd(qd, kd, vd, causal=causal, mask=dm)
        seen.add(abi.sdpa_last_kernel())
        q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
        want = torch.softmax(scores64(q64, k64, causal, mask), -1) @ v64.repeat_interleave(Hq // Hkv, 1)
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        err = (got.cpu().double() - want.detach()).abs().max().item()
        assert err <= tol, f"{tag}: forward max-abs {err:.3e} on {abi.sdpa_last_kernel()}"

        want.backward(do.double())
        if mask is None and dtype != torch.float32 and D % 8 == 0 and (D in (64, 128) or Lk % 8 == 0):
            o, lse = abi.sdpa_fwd(qd, kd, vd, causal=causal, return_lse=True)
            grads = abi.sdpa_bwd(do.to(DEV), qd, kd, vd, o, lse, causal=causal)
        else:
            grads = abi.sdpa_bwd_general(do.to(DEV), qd, kd, vd, causal=causal, mask=dm)
        for got_g, want_g, name in zip(grads, (q64.grad, k64.grad, v64.grad), ("dq", "dk", "dv")):
            scale = max(want_g.abs().max().item(), 1e-2)      # a row that sees one key has gradient zero
            rel = (got_g.cpu().double() - want_g).abs().max().item() / scale
            assert rel <= (2e-4 if dtype == torch.float32 else 2e-2), f"{tag}: {name} off by {rel:.3e} of its scale"
    assert {"tcgen05", "simt"} <= seen, seen


@pytest.mark.parametrize("seed", [21, 22])
def test_random_long_key_ranges(seed):
    """Few query blocks against long key ranges, the shapes whose key range the tensor-core kernel cuts
    into pieces: forward, the log-sum-exp the pieces are merged with, and the fused backward fed by it."""
    rnd = random.Random(seed)
    for it in range(16):
        dtype = rnd.choice([torch.bfloat16, torch.float16])
        D = rnd.choice([128, 128, 64])
        Hkv = rnd.choice([1, 2])
        Hq = Hkv * rnd.choice([1, 2, 4])
        B = rnd.choice([1, 2])
        Lq = rnd.choice([17, 64, 128, 200, 300, 520, 1100])
        Lk = rnd.choice([1000, 1500, 2047, 2048, 3000, 4100])
        causal = rnd.random() < 0.3
        g = torch.Generator().manual_seed(seed * 1000 + it)
        q = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
        k = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
        v = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
        do = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
        tag = f"seed {seed} case {it}: {dtype} B{B} Hq{Hq} Hkv{Hkv} Lq{Lq} Lk{Lk} D{D} causal={causal}"
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
        o, lse = abi.sdpa_fwd(qd, kd, vd, causal=causal, return_lse=True, flags=abi.SDPA_FORCE_TENSOR)
        q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
        s = scores64(q64, k64, causal, None)
        want = torch.softmax(s, -1) @ v64.repeat_interleave(Hq // Hkv, 1)
        err = (o.cpu().double() - want.detach()).abs().max().item()
        assert err <= 2e-2, f"{tag}: forward max-abs {err:.3e}"
        lerr = (lse.cpu().double() - torch.logsumexp(s.detach(), -1)).abs().max().item()
        assert lerr <= 2e-3, f"{tag}: lse off by {lerr:.3e}"
        want.backward(do.double())
        grads = abi.sdpa_bwd(do.to(DEV), qd, kd, vd, o, lse, causal=causal)
        for got_g, want_g, name in zip(grads, (q64.grad, k64.grad, v64.grad), ("dq", "dk", "dv")):
            scale = max(want_g.abs().max().item(), 1e-2)
            rel = (got_g.cpu().double() - want_g).abs().max().item() / scale
            assert rel <= 2e-2, f"{tag}: {name} off by {rel:.3e} of its scale"
