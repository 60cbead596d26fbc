"""GPU parity tests proper: the CUDA kernels, called through the C ABI (ctypes on
libparas_b200.so with raw device pointers), against the CPU oracle and the committed golden
vectors of the reference build.

Tolerances (stated by the task): fp32 max-abs 1e-4 (checked as the reference's own
atol = rtol = 1e-4); bf16 / fp16 max-abs 2e-2 with fp32 accumulation.
"""
import math

import pytest
import torch

from conftest import golden_names, load_golden
from oracle import oracle as O
from oracle import stats

import torch_paras  # noqa: F401
from torch_paras import abi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def tol_check(got, want, name=""):
    got = got.detach().cpu()
    assert got.dtype == want.dtype, f"{name}: dtype {got.dtype} vs {want.dtype}"
    assert got.shape == want.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if want.dtype == torch.float32:
        ok = torch.allclose(got, want, atol=1e-4, rtol=1e-4, equal_nan=True)
        err = (got.double() - want.double()).abs().max().item() if got.numel() else 0.0
        assert ok, f"{name}: fp32 mismatch, max-abs {err:.3e}"
    else:
        r = stats.report(got, want, 2e-2)   # max-abs, count over 2e-2, share within 1 ulp
        print(f"{name}: {stats.fmt(r)}")
        assert r["over_tol"] == 0 and r["max_abs"] <= 2e-2, f"{name}: 16-bit mismatch, {stats.fmt(r)}"
    return None


def run_cuda(op, a, **kw):
    c = lambda t: t.to(DEV) if torch.is_tensor(t) else t  # noqa: E731
    if op == "sdpa":
        q, k, v = c(a["q"]), c(a["k"]), c(a["v"])
        return abi.sdpa_fwd(q, k, v, causal=bool(a.get("is_causal", False)), scale=a.get("scale"),
                            mask=c(a.get("attn_mask")), flags=abi.SDPA_REF_SCALE | kw.get("flags", 0))
    if op == "sdpa_math":   # (output, weights after dropout) with the reference's Philox stream re-seeded
        q, k, v = c(a["q"]), c(a["k"]), c(a["v"])
        return abi.sdpa_fwd(q, k, v, causal=bool(a.get("is_causal", False)), scale=a.get("scale"),
                            mask=c(a.get("attn_mask")), flags=abi.SDPA_REF_SCALE,
                            dropout_p=float(a.get("dropout_p", 0.0)), rng=(int(a.get("seed", 0)), 0),
                            dropout_mask=c(a.get("dropout_mask")), return_weights=True)
    if op == "rms_norm_aten":
        x = c(a["x"])
        n = 1
        for s in a["normalized_shape"]:
            n *= s
        w = c(a["weight"]).reshape(n) if a.get("weight") is not None else None
        eps = 1e-6 if a.get("eps") is None else a["eps"]
        return abi.rmsnorm_fwd(x.reshape(-1, n), w, eps, mode=abi.ROUND_PER_OP).reshape(x.shape)
    if op == "rms_norm_paras":
        return abi.rmsnorm_fwd(c(a["x"]), c(a["weight"]), a["eps"], return_rstd=True)
    if op == "rms_norm_paras_backward":
        return abi.rmsnorm_bwd(c(a["grad_out"]), c(a["x"]), c(a["weight"]), c(a["rstd"]))
    if op == "swiglu_paras":
        return abi.swiglu_fwd(c(a["gate"]), c(a["up"]))
    if op == "swiglu_paras_backward":
        return abi.swiglu_bwd(c(a["grad_out"]), c(a["gate"]), c(a["up"]))
    if op == "swiglu_composite":
        return abi.swiglu_fwd(c(a["gate"]), c(a["x"]), mode=abi.ROUND_PER_OP)
    if op == "rotate_half":
        return abi.rotate_half(c(a["x"]))
    if op == "rotate_half_backward":
        return abi.rotate_half(c(a["grad_out"]), backward=True)
    if op == "rope_sdpa":   # (rotated q, rotated k, attention over them): rotation alone, then the fused call
        q, k, v, cos, sin = c(a["q"]), c(a["k"]), c(a["v"]), c(a["cos"]), c(a["sin"])
        pos0 = int(a.get("q_pos0", 0))
        out = abi.sdpa_rope_fwd(q, k, v, cos, sin, q_pos0=pos0, causal=bool(a.get("is_causal", False)),
                                flags=abi.SDPA_REF_SCALE)
        return abi.rope(q, cos, sin, pos0=pos0), abi.rope(k, cos, sin, pos0=0), out
    raise AssertionError(op)


def as_tuple(x):
    return x if isinstance(x, tuple) else (x,)


@pytest.mark.parametrize("name", golden_names())
def test_against_reference_golden_vectors(name):
    g = load_golden(name)
    got = as_tuple(run_cuda(g["op"], g["args"]))
    want = as_tuple(g["out"])
    for i, (a, b) in enumerate(zip(got, want)):
        if g["op"] == "rope_sdpa" and i < 2:   # the rotation is three rounded element-wise steps: exact
            assert torch.equal(a.cpu(), b), f"{name}[{i}]: rotated tensor differs from the reference's"
        else:
            tol_check(a, b, f"{name}[{i}]")


def _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Lq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
    return q, k, v


SDPA_CASES = [
    # B, Hq, Hkv, Lq,  Lk,  D,  causal
    (1, 2, 2, 256, 256, 128, True),     # exactly one CTA of two query tiles
    (2, 4, 4, 512, 512, 128, True),
    (1, 8, 2, 640, 640, 128, True),     # GQA 4:1, odd number of query tiles
    (1, 4, 1, 300, 300, 128, True),     # ragged: not a multiple of any tile
    (1, 2, 2, 384, 384, 128, False),    # full attention
    (1, 2, 2, 200, 456, 128, False),    # Lq != Lk, ragged
    (1, 2, 2, 130, 400, 128, True),     # causal with Lk > Lq: top-left alignment
    (1, 2, 2, 400, 130, 128, True),     # causal with Lk < Lq
    (2, 8, 2, 1, 700, 128, False),      # decode step, GQA
    (2, 8, 2, 2, 900, 64, False),       # decode step with head dim 64 (the decode kernel's one-slab form)
    (1, 4, 4, 7, 260, 128, False),      # a few query rows
    (1, 2, 2, 129, 129, 64, True),      # D = 64
    (2, 4, 2, 640, 640, 64, True),      # D = 64 on the tensor-core kernel: GQA, several kv tiles
    (1, 2, 2, 300, 456, 64, False),     # D = 64, ragged, Lq != Lk
    (1, 3, 1, 50, 77, 32, False),       # small D, GQA 3:1
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("case", SDPA_CASES)
def test_sdpa_against_oracle(case, dtype):
    B, Hq, Hkv, Lq, Lk, D, causal = case
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=hash(case) % 10000)
    want = O.sdpa(q, k, v, is_causal=causal, enable_gqa=Hq != Hkv)
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=causal, flags=abi.SDPA_REF_SCALE)
    tol_check(got, want, f"sdpa {case} {dtype} [{abi.sdpa_last_kernel()}]")


def test_split_kv_with_odd_head_dim_and_odd_split_count():
    # D = 63 with one query row and 5 key ranges: 315 fp32 partials, after which the {max, sum}
    # pairs used to land on a 4-byte boundary
    q, k, v = _qkv(1, 1, 1, 1, 1280, 63, torch.float32, seed=63)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    got = abi.sdpa_fwd(qd, kd, vd, flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel() == "simt_splitkv"
    tol_check(got, O.sdpa(q, k, v), "odd D split-KV")
    got2 = abi.sdpa_fwd_static_scratch(qd, kd, vd, flags=abi.SDPA_REF_SCALE)
    tol_check(got2, O.sdpa(q, k, v), "odd D split-KV, static scratch")
    for D, Lk in ((33, 2000), (1, 1500), (255, 1100)):
        q, k, v = _qkv(1, 3, 1, 1, Lk, D, torch.bfloat16, seed=D)
        got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), flags=abi.SDPA_REF_SCALE)
        tol_check(got, O.sdpa(q, k, v, enable_gqa=True), f"odd D={D} split-KV bf16")


def test_a_bounded_wait_that_runs_out_is_reported_once_and_the_gpu_stays_usable():
    # A one-warp kernel waits (with the primitive all tensor-core kernels wait with) on a barrier
    # nobody arrives at, limit 1 ms: it gives up and returns by itself.  The host sees
    # PARAS_E_TIMEOUT with the wait's bit in the status word, once; the launches that follow --
    # attention and the GEMM share that status word -- run and give correct results.
    st, word = abi.selftest_bounded_wait(0, 1000)
    assert st == -6, abi.lib().paras_b200_last_error()
    assert word & 0x40000000 and word & (1 << 27), hex(word & 0xffffffff)
    assert b"gave up a bounded wait" in abi.lib().paras_b200_last_error()
    assert abi.lib().paras_b200_synchronize(0) == 0          # reported once, not again
    q, k, v = _qkv(1, 2, 2, 512, 512, 128, torch.bfloat16, 5)
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=True, flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    tol_check(got, O.sdpa(q, k, v, is_causal=True), "attention after a reported timeout")
    a = torch.randn(256, 256, device=DEV).bfloat16()
    c = abi.gemm(a, a)
    assert torch.allclose(c.float(), a.float() @ a.float().t(), rtol=2.0 ** -7, atol=0.1)  # one bf16 ulp
    # a failure noticed by another entry point (here: synchronize) does not poison later launches
    st, _ = abi.selftest_bounded_wait(0, 200)
    assert st == -6
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=True, flags=abi.SDPA_REF_SCALE)
    tol_check(got, O.sdpa(q, k, v, is_causal=True), "attention after a second reported timeout")


DECODE_CASES = [
    # B, Hq, Hkv, Lq, Lk, causal
    (2, 8, 2, 1, 4096, False),      # group of 4, one query position
    (1, 16, 1, 1, 5000, False),     # 16 query heads on one kv head; cache not a multiple of the tile
    (3, 8, 4, 2, 1031, False),      # two query positions x group of 2
    (1, 8, 2, 4, 777, True),        # causal, top-left aligned: position i sees keys 0..i only
    (1, 4, 4, 3, 9000, False),      # no sharing (group 1), three positions, several key ranges
    (1, 2, 1, 1, 40000, False),     # long cache, few units: many key ranges per kv head
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", DECODE_CASES)
def test_decode_kernel_against_oracle(case, dtype):
    B, Hq, Hkv, Lq, Lk, causal = case
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, 128, dtype, seed=Lk)
    want = O.sdpa(q, k, v, is_causal=causal, enable_gqa=Hq != Hkv)
    got, lse = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=causal, flags=abi.SDPA_REF_SCALE,
                            return_lse=True)
    assert abi.sdpa_last_kernel() == "decode_mma"
    tol_check(got, want, f"decode {case} {dtype}")
    ref = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=causal, return_lse=True,
                       flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_SIMT)
    assert torch.allclose(lse, ref[1], atol=2e-3, rtol=2e-3)


def test_decode_kernel_strided_cache_and_workspace():
    # K/V cache stored [B, L, Hkv, D] (token-major, as a paged cache would hand it over)
    g = torch.Generator().manual_seed(77)
    ks = torch.randn(2, 3000, 2, 128, generator=g).bfloat16()
    vs = torch.randn(2, 3000, 2, 128, generator=g).bfloat16()
    q = torch.randn(2, 8, 1, 128, generator=g).bfloat16()
    want = O.sdpa(q, ks.transpose(1, 2), vs.transpose(1, 2), enable_gqa=True)
    kd, vd, qd = ks.to(DEV).transpose(1, 2), vs.to(DEV).transpose(1, 2), q.to(DEV)
    need = abi.sdpa_workspace_bytes(qd, kd, vd)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    got = abi.sdpa_fwd(qd, kd, vd, flags=abi.SDPA_REF_SCALE, workspace=ws)
    assert abi.sdpa_last_kernel() == "decode_mma"
    tol_check(got, want, "strided decode")
    if need:
        with pytest.raises(RuntimeError, match="smaller than"):
            abi.sdpa_fwd(qd, kd, vd, workspace=ws[:16])


def test_tensor_core_kernel_is_the_one_that_runs():
    q, k, v = _qkv(1, 2, 2, 512, 512, 128, torch.bfloat16, 5)
    abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=True)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    q32 = q.float()
    abi.sdpa_fwd(q32.to(DEV), k.float().to(DEV), v.float().to(DEV), causal=True)
    assert abi.sdpa_last_kernel().startswith("simt")


def test_sdpa_simt_and_tensor_kernels_agree():
    q, k, v = _qkv(1, 4, 2, 700, 700, 128, torch.bfloat16, 11)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    a = abi.sdpa_fwd(qd, kd, vd, causal=True)
    b = abi.sdpa_fwd(qd, kd, vd, causal=True, flags=abi.SDPA_FORCE_SIMT)
    assert (a.float() - b.float()).abs().max().item() <= 2e-2


SPLIT_KEY_CASES = [
    # B, Hq, Hkv, Lq,  Lk,   D,  causal: few query blocks against many keys on the tensor-core kernel
    (1, 8, 2, 300, 5000, 128, False),     # a prompt chunk over a long cache, GQA, ragged both ways
    (2, 4, 4, 64, 4096, 64, False),       # D = 64, one query tile
    (1, 4, 4, 1500, 3000, 128, True),     # causal: later key ranges hold only the later query tiles
    (1, 2, 1, 520, 2100, 128, False),     # three query blocks (the middle one has no partner)
    (1, 3, 3, 17, 8200, 128, False),      # more rows than the decode kernel takes
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", SPLIT_KEY_CASES)
def test_split_keys_on_the_tensor_core_kernel(case, dtype):
    # Too few (batch, head, query block) units to fill the GPU: the key range is cut into pieces that
    # run as separate units, and a second kernel merges the partial outputs by their log-sum-exp.
    B, Hq, Hkv, Lq, Lk, D, causal = case
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=hash(case) % 10000)
    want = O.sdpa(q, k, v, is_causal=causal, enable_gqa=Hq != Hkv)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    got, lse = abi.sdpa_fwd(qd, kd, vd, causal=causal, return_lse=True, flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    need = abi.sdpa_workspace_bytes(qd, kd, vd, causal=causal, flags=abi.SDPA_FORCE_TENSOR)
    assert need > 0, "this shape was meant to take the split-key route"
    tol_check(got, want, f"split keys {case} {dtype}")
    sc = float(torch.tensor(1 / math.sqrt(D)).to(dtype))
    kk = k.repeat_interleave(Hq // Hkv, 1)
    s = (q.double() @ kk.double().transpose(-1, -2)) * sc
    if causal:
        s = s.masked_fill(~torch.ones(Lq, Lk, dtype=torch.bool).tril(), float("-inf"))
    assert torch.allclose(lse.cpu().double(), torch.logsumexp(s, -1), atol=2e-3, rtol=2e-3)
    # caller-owned scratch gives the same bits, and a scratch that is too small is refused
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    assert torch.equal(abi.sdpa_fwd(qd, kd, vd, causal=causal, workspace=ws, flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR), got)
    with pytest.raises(RuntimeError):
        abi.sdpa_fwd(qd, kd, vd, causal=causal, workspace=ws[:need // 2], flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR)


PACKED_CASES = [
    # B, Hq, Hkv, Lq, Lk,  D,  causal, expected route: a few query positions of a whole GQA group in one item
    (2, 8, 2, 64, 700, 128, False, "tcgen05_packed"),          # 4 heads x 64 rows
    (1, 8, 1, 32, 5000, 128, False, "tcgen05_packed_split"),   # 8 heads x 32 rows, long key range
    (2, 4, 2, 128, 300, 64, True, "tcgen05_packed"),           # 2 heads x 128 rows, causal, D = 64
    (1, 8, 2, 40, 3000, 128, True, "tcgen05_packed"),          # causal with Lk > Lq: 40 visible keys at most
    (3, 16, 4, 17, 700, 64, False, "tcgen05_packed"),          # rows past Lq inside every head's slot
    (1, 16, 2, 20, 9000, 128, False, "tcgen05_packed_split"),
    (1, 4, 2, 100, 2500, 128, False, "tcgen05_packed_split"),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", PACKED_CASES)
def test_packed_gqa_groups_on_the_tensor_core_kernel(case, dtype):
    B, Hq, Hkv, Lq, Lk, D, causal, route = case
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=hash(case) % 10000)
    want = O.sdpa(q, k, v, is_causal=causal, enable_gqa=True)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    got, lse = abi.sdpa_fwd(qd, kd, vd, causal=causal, return_lse=True, flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR)
    assert abi.sdpa_last_kernel() == route
    tol_check(got, want, f"packed groups {case} {dtype}")
    sc = float(torch.tensor(1 / math.sqrt(D)).to(dtype))
    s = (q.double() @ k.repeat_interleave(Hq // Hkv, 1).double().transpose(-1, -2)) * sc
    if causal:
        s = s.masked_fill(~torch.ones(Lq, Lk, dtype=torch.bool).tril(), float("-inf"))
    assert torch.allclose(lse.cpu().double(), torch.logsumexp(s, -1), atol=2e-3, rtol=2e-3)
    # q as a [B, L, H, D] projection output viewed as [B, H, L, D]; output into the same layout
    qs = q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    out = torch.empty(B, Lq, Hq, D, dtype=dtype, device=DEV).transpose(1, 2)
    abi.sdpa_fwd(qs, kd, vd, causal=causal, out=out, flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR)
    assert torch.equal(out, got)


def test_sdpa_strided_inputs_and_lse():
    # [B, L, H, D] storage viewed as [B, H, L, D]: what a fused QKV projection produces
    g = torch.Generator().manual_seed(3)
    qs = torch.randn(2, 300, 4, 128, generator=g).bfloat16()
    ks = torch.randn(2, 300, 4, 128, generator=g).bfloat16()
    vs = torch.randn(2, 300, 4, 128, generator=g).bfloat16()
    q, k, v = (t.transpose(1, 2) for t in (qs, ks, vs))
    want = O.sdpa(q, k, v, is_causal=True)
    got, lse = abi.sdpa_fwd(qs.to(DEV).transpose(1, 2), ks.to(DEV).transpose(1, 2),
                            vs.to(DEV).transpose(1, 2), causal=True, return_lse=True,
                            flags=abi.SDPA_REF_SCALE)
    tol_check(got, want, "strided sdpa")
    sc = float(torch.tensor(1 / math.sqrt(128)).bfloat16())
    s = (q.float() @ k.float().transpose(-1, -2)) * sc
    s = s.masked_fill(~torch.ones(300, 300, dtype=torch.bool).tril(), float("-inf"))
    assert torch.allclose(lse.cpu(), torch.logsumexp(s, -1), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("factor", [3.0, 6.0, 30.0, 200.0])
def test_sdpa_scores_that_grow_from_tile_to_tile(factor, causal, dtype):
    # Every third 128-key tile has keys scaled up, more so the later it comes, so a row's
    # largest score keeps moving as the kernel walks the keys: by a little (the reference of
    # the online softmax moves lazily), and by far more than the exponent range of the
    # probabilities (the tile has to be redone against its own max).
    B, Hq, Hkv, L = 1, 2, 1, 1024
    q, k, v = _qkv(B, Hq, Hkv, L, L, 128, dtype, seed=17)
    for j in range(L // 128):
        if j % 3 == 2:
            k[:, :, 128 * j:128 * (j + 1)] *= factor * (1 + j) / 8.0
    # Checked against float64 attention, not against the reference's numerics: the reference
    # rounds the scores to 16 bits before the softmax (attention_ops.cpp:96-118), which at
    # scores of this size (tens to thousands) is an error of whole units in the exponent.
    got, lse = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=causal, return_lse=True,
                            flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    sc = float(torch.tensor(1 / math.sqrt(128)).to(dtype))
    s = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc
    if causal:
        s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool).tril(), float("-inf"))
    want = torch.softmax(s, -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
    g = got.cpu().double()
    assert torch.isfinite(g).all()
    # 2e-2 relative to max(1, |want|): the softmax is nearly one-hot for the larger factors, so
    # outputs are single V entries of size up to 4 and more (one bf16 ulp at 4 is 3.1e-2)
    err = ((g - want).abs() / want.abs().clamp(min=1.0)).max().item()
    assert err <= 2e-2, f"growing scores x{factor} causal={causal} {dtype}: {err:.3e}"
    assert torch.allclose(lse.cpu().double(), torch.logsumexp(s, -1), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["bool_padding", "bool_blocks", "additive_same", "additive_f32", "ragged_bool",
                                  "additive_ragged_rows"])
def test_tensor_core_kernel_with_explicit_masks(kind, dtype):
    # attn_mask on the tcgen05 path (16 bit, D = 128): bool and additive, broadcast strides,
    # vector and element-wise reads, rows whose first key tiles are masked out entirely, and rows
    # with no key at all (NaN, as in the reference)
    B, Hq, Hkv = 2, 4, 2
    # (contiguous, 16-byte aligned mask rows are read by the warp as a block; "additive_ragged_rows"
    # takes that path with a last query tile that ends at row 300 of 384)
    Lq, Lk = (300, 333) if kind == "ragged_bool" else ((300, 512) if kind == "additive_ragged_rows" else (384, 512))
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, 128, dtype, seed=23)
    g = torch.Generator().manual_seed(29)
    if kind == "bool_padding":      # per batch element: keys past its length are padding
        lens = [Lk, 200]
        mask = torch.zeros(B, 1, 1, Lk, dtype=torch.bool)
        for b, n in enumerate(lens):
            mask[b, :, :, :n] = True
    elif kind == "bool_blocks":     # rows see a window that starts after the first key tile(s)
        mask = torch.zeros(1, 1, Lq, Lk, dtype=torch.bool)
        for r in range(Lq):
            lo = 130 + (r % 7) * 40
            mask[0, 0, r, lo:lo + 60] = True
        mask[0, 0, 5] = False        # a row without any key
        mask[0, 0, 200] = False
    elif kind in ("additive_same", "additive_ragged_rows"):
        mask = (torch.randn(Lq, Lk, generator=g) * 2).to(dtype)
    elif kind == "additive_f32":
        mask = torch.randn(B, Hq, Lq, Lk, generator=g) * 2
        mask[:, :, :, 100:160] = float("-inf")
    else:
        mask = torch.rand(B, Hq, Lq, Lk, generator=g) > 0.3
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=mask.to(DEV), flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    if mask.dtype == torch.bool:
        tol_check(got, O.sdpa(q, k, v, attn_mask=mask, enable_gqa=True), f"masked sdpa {kind} {dtype}")
    else:
        # The reference adds the mask to scores it has already rounded to 16 bits and rounds the sum
        # again (attention_ops.cpp:96-126): with mask values of several units that is an error of
        # a few percent in the probabilities.  The kernel keeps the sum in fp32, so it is checked
        # against float64 attention on the same 16-bit inputs.
        sc = float(torch.tensor(1 / math.sqrt(128)).to(dtype))
        s = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc + mask.double()
        want = torch.softmax(s, -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
        assert (got.cpu().double() - want).abs().max().item() <= 2e-2, f"masked sdpa {kind} {dtype}"
    simt = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=mask.to(DEV),
                        flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_SIMT)
    assert torch.equal(torch.isnan(got), torch.isnan(simt))
    assert (got.float() - simt.float()).nan_to_num(0.0).abs().max().item() <= 2e-2


def test_head_dim_64_runs_on_the_tensor_core_kernel_with_masks_and_lse():
    q, k, v = _qkv(2, 4, 2, 333, 400, 64, torch.bfloat16, seed=31)
    mask = torch.rand(2, 1, 333, 400, generator=torch.Generator().manual_seed(5)) > 0.4
    want = O.sdpa(q, k, v, attn_mask=mask, enable_gqa=True)
    got, lse = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=mask.to(DEV), return_lse=True,
                            flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel().startswith("tcgen05")
    tol_check(got, want, "D=64 masked")
    sc = float(torch.tensor(1 / math.sqrt(64)).bfloat16())
    s = (q.float() @ k.float().repeat_interleave(2, 1).transpose(-1, -2)) * sc
    s = s.masked_fill(~mask, float("-inf"))
    assert torch.allclose(lse.cpu(), torch.logsumexp(s, -1), atol=2e-3, rtol=2e-3)


def test_sdpa_empty_and_degenerate_shapes():
    z = torch.empty(1, 2, 0, 128, dtype=torch.bfloat16, device=DEV)
    kv = torch.randn(1, 2, 16, 128, device=DEV).bfloat16()
    assert abi.sdpa_fwd(z, kv, kv).shape == (1, 2, 0, 128)
    q = torch.randn(1, 2, 4, 128, device=DEV).bfloat16()
    no_keys = torch.empty(1, 2, 0, 128, dtype=torch.bfloat16, device=DEV)
    out = abi.sdpa_fwd(q, no_keys, no_keys)          # softmax over nothing, times nothing = 0
    assert torch.equal(out.cpu(), torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16))
    # a row whose keys are all masked out is NaN in the reference too
    mask = torch.ones(1, 1, 4, 16, dtype=torch.bool)
    mask[0, 0, 2] = False
    want = O.sdpa(q.cpu(), kv.cpu(), kv.cpu(), attn_mask=mask)
    got = abi.sdpa_fwd(q, kv, kv, mask=mask.to(DEV), flags=abi.SDPA_REF_SCALE)
    tol_check(got, want, "fully masked row")
    with pytest.raises(RuntimeError, match="mutually exclusive"):
        abi.sdpa_fwd(q, kv, kv, causal=True, mask=mask.to(DEV))
    with pytest.raises(RuntimeError, match="multiple of key/value heads"):
        abi.sdpa_fwd(torch.randn(1, 5, 4, 8, device=DEV), torch.randn(1, 2, 4, 8, device=DEV),
                     torch.randn(1, 2, 4, 8, device=DEV))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(64, 4096), (33, 1024), (7, 100), (3, 8200), (5, 24), (0, 16), (130, 256)])
def test_rmsnorm_both_entry_points_against_oracle(shape, dtype):
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    x = torch.randn(*shape, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(shape[1], generator=g)).to(dtype)
    y, rstd = abi.rmsnorm_fwd(x.to(DEV), w.to(DEV), 1e-6, return_rstd=True)
    yo, ro = O.rms_norm_fused(x, w, 1e-6)
    tol_check(y, yo, "paras::rms_norm")
    assert torch.allclose(rstd.cpu(), ro, atol=1e-6, rtol=1e-5)
    if dtype != torch.float32 and shape[0]:
        frac = (y.cpu() == yo).float().mean().item()
        assert frac > 0.999, f"fused RMSNorm only {frac:.4f} bit-exact"
    yc = abi.rmsnorm_fwd(x.to(DEV), w.to(DEV), 1e-6, mode=abi.ROUND_PER_OP)
    yco = O.rms_norm_composite(x, [shape[1]], w, 1e-6)
    tol_check(yc, yco, "aten::rms_norm")
    if dtype != torch.float32 and shape[0]:
        frac = (yc.cpu() == yco).float().mean().item()
        assert frac > 0.99, f"per-op-rounding RMSNorm only {frac:.4f} bit-exact"
    yn = abi.rmsnorm_fwd(x.to(DEV), None, 1e-5, mode=abi.ROUND_PER_OP)
    tol_check(yn, O.rms_norm_composite(x, [shape[1]], None, 1e-5), "aten::rms_norm no weight")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("n", [(128, 14336), (17, 77), (1, 1), (0, 4), (3, 1000003)])
def test_swiglu_both_entry_points_against_oracle(n, dtype):
    g = torch.Generator().manual_seed(n[0] + n[1])
    gate = torch.randn(*n, generator=g).to(dtype)
    up = torch.randn(*n, generator=g).to(dtype)
    tol_check(abi.swiglu_fwd(gate.to(DEV), up.to(DEV)), O.swiglu_fused(gate, up), "paras::swiglu")
    tol_check(abi.swiglu_fwd(gate.to(DEV), up.to(DEV), mode=abi.ROUND_PER_OP),
              O.swiglu_composite(up, gate), "torch_paras::swiglu")
    if dtype == torch.bfloat16 and gate.numel():
        frac = (abi.swiglu_fwd(gate.to(DEV), up.to(DEV)).cpu() == O.swiglu_fused(gate, up)).float().mean().item()
        assert frac > 0.999


def test_swiglu_unaligned_pointers_take_the_scalar_path():
    g = torch.Generator().manual_seed(4)
    gate = torch.randn(4099, generator=g).bfloat16()
    up = torch.randn(4099, generator=g).bfloat16()
    gd, ud = gate.to(DEV)[1:], up.to(DEV)[1:]          # 2-byte offset: not 16-byte aligned
    out = torch.empty_like(gd)
    abi.swiglu_fwd(gd, ud, out=out)
    tol_check(out, O.swiglu_fused(gate[1:], up[1:]), "unaligned swiglu")


def test_backward_ops_and_rotate_half_against_oracle():
    g = torch.Generator().manual_seed(8)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(37, 200, generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(200, generator=g)).to(dtype)
        go = torch.randn(37, 200, generator=g).to(dtype)
        _, rstd = O.rms_norm_fused(x, w, 1e-6)
        gx, gw = abi.rmsnorm_bwd(go.to(DEV), x.to(DEV), w.to(DEV), rstd.to(DEV))
        gxo, gwo = O.rms_norm_fused_backward(go, x, w, rstd)
        tol_check(gx, gxo, "rms_norm_backward dx")
        if dtype == torch.float32:
            tol_check(gw, gwo, "rms_norm_backward dw")
        else:
            assert (gw.cpu().double() - gwo.double()).abs().max().item() <= 2e-2 * max(1.0, gwo.abs().max().item())
        gate = torch.randn(19, 33, generator=g).to(dtype)
        up = torch.randn(19, 33, generator=g).to(dtype)
        d = torch.randn(19, 33, generator=g).to(dtype)
        gg, gu = abi.swiglu_bwd(d.to(DEV), gate.to(DEV), up.to(DEV))
        ggo, guo = O.swiglu_fused_backward(d, gate, up)
        tol_check(gg, ggo, "swiglu_backward dgate")
        tol_check(gu, guo, "swiglu_backward dup")
        r = torch.randn(5, 64, generator=g).to(dtype)
        assert torch.equal(abi.rotate_half(r.to(DEV)).cpu(), O.rotate_half(r))
        assert torch.equal(abi.rotate_half(r.to(DEV), backward=True).cpu(), O.rotate_half_backward(r))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [
    (1300, 4096),    # ring in shared memory, two rows a step
    (2500, 1024),    # four rows a step
    (700, 7168),     # the last vector slot of some threads lies past the row
    (650, 5120),
    (333, 8192),     # 256 / 512 threads
    (301, 16384),
    (100, 4096),     # too few rows for the ring: the plain one-pass kernel
    (1300, 4104),    # a row length that no CTA size divides
    (41, 1000),      # rows that are not whole 16-byte vectors in fp16/bf16 ... the two-kernel route
    (1187, 2048),    # an odd row count: the last step of some CTAs is half empty
])
def test_rmsnorm_backward_row_kernels_against_oracle(shape, dtype):
    rows, H = shape
    g = torch.Generator().manual_seed(rows + H)
    x = torch.randn(rows, H, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    go = torch.randn(rows, H, generator=g).to(dtype)
    _, rstd = O.rms_norm_fused(x, w, 1e-6)
    gx, gw = abi.rmsnorm_bwd(go.to(DEV), x.to(DEV), w.to(DEV), rstd.to(DEV))
    gxo, gwo = O.rms_norm_fused_backward(go, x, w, rstd)
    tol_check(gx, gxo, f"rms_norm_backward dx {shape}")
    # grad_weight sums `rows` products per column: the oracle adds them in the tensors' order in fp32, the
    # kernel per CTA in fp32 and across CTAs in double; both round once at the end
    ref = (go.double() * x.double() * rstd.double()[:, None]).sum(0)
    err = (gw.cpu().double() - ref).abs().max().item()
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else (2.0 ** -11 if dtype == torch.float16 else 2.0 ** -20)
    assert err <= ulp * max(1.0, ref.abs().max().item()) + 1e-3, f"dw {shape}: {err:.3e}"
    assert (gw.cpu().double() - gwo.double()).abs().max().item() <= 2e-2 * max(1.0, gwo.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["bool", "additive", "additive_f32", "bool_4d", "additive_min"])
@pytest.mark.parametrize("shape", [(640, 640), (300, 456), (456, 300)])
def test_a_causal_mask_written_out_runs_as_the_causal_kernel(shape, kind, dtype):
    # attn_mask = the lower triangle as a tensor (bool, or 0 / -inf): a check kernel recognises it and the
    # masked kernel then skips the tiles above the diagonal and never reads the mask; one entry off the
    # pattern and the mask is applied as given.  Both against the oracle, and against is_causal=True.
    Lq, Lk = shape
    q, k, v = _qkv(2, 4, 2, Lq, Lk, 128, dtype, seed=91)
    tri = torch.ones(Lq, Lk, dtype=torch.bool).tril()
    def as_kind(t):
        if kind == "bool":
            return t
        if kind == "bool_4d":
            return t[None, None]
        if kind == "additive_min":     # the most negative finite value instead of -inf, as some callers write it
            return torch.zeros(Lq, Lk, dtype=dtype).masked_fill(~t, torch.finfo(dtype).min)
        m = torch.zeros(Lq, Lk).masked_fill(~t, float("-inf"))
        return m.to(dtype) if kind == "additive" else m
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    flags = abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR
    got = abi.sdpa_fwd(qd, kd, vd, mask=as_kind(tri).to(DEV), flags=flags)
    assert abi.sdpa_last_kernel() == "tcgen05"
    tol_check(got, O.sdpa(q, k, v, is_causal=True, enable_gqa=True), f"written-out causal {kind} {shape}")
    assert torch.equal(got, abi.sdpa_fwd(qd, kd, vd, causal=True, flags=flags))
    off = tri.clone()
    off[Lq // 2, min(Lk - 1, Lq // 2 + 3)] = True        # one key above the diagonal is visible
    off[Lq - 1, 0] = False                                # and one below it is not
    got2 = abi.sdpa_fwd(qd, kd, vd, mask=as_kind(off).to(DEV), flags=flags)
    if kind.startswith("bool"):
        want2 = O.sdpa(q, k, v, attn_mask=off, enable_gqa=True)
        tol_check(got2, want2, f"almost causal {kind} {shape}")
    else:
        sc = float(torch.tensor(1 / math.sqrt(128)).to(dtype))
        s_ = (q.double() @ k.double().repeat_interleave(2, 1).transpose(-1, -2)) * sc
        s_ = s_.masked_fill(~off, float("-inf"))
        want2 = torch.softmax(s_, -1) @ v.double().repeat_interleave(2, 1)
        assert (got2.cpu().double() - want2).abs().max().item() <= 2e-2
    assert not torch.equal(got2, got)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["bool", "additive_min", "additive_f32", "left_padded", "one_off"])
@pytest.mark.parametrize("shape", [(640, 640), (300, 456)])
def test_causal_masks_over_right_padded_sequences_run_as_causal_with_lengths(shape, kind, dtype):
    # [B, 1, Lq, Lk] masks built as (key <= query) & (key < len_b): what callers pass for a padded batch when
    # they cannot use is_causal.  A check kernel finds len_b and verifies every entry; the masked kernel then
    # skips the tiles above the diagonal and past len_b and never reads the mask.  Left padding or one entry
    # off the pattern and the mask is applied as given.
    Lq, Lk = shape
    B, Hq, Hkv, D = 4, 4, 2, 128
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=95)
    lens = (min(Lq, Lk), 300, 129, 1)
    tri = torch.ones(Lq, Lk, dtype=torch.bool).tril()
    vis = torch.stack([tri & (torch.arange(Lk)[None, :] < n) for n in lens])[:, None]        # [B,1,Lq,Lk]
    if kind == "left_padded":
        vis = torch.stack([tri & (torch.arange(Lk)[None, :] >= Lk // 4) for _ in lens])[:, None]
        vis[..., 0] |= ~vis.any(-1)             # no empty rows
    if kind == "one_off":
        vis = vis.clone()
        vis[1, 0, Lq // 2, 3] = False
    if kind in ("bool", "left_padded", "one_off"):
        given = vis
    elif kind == "additive_min":
        given = torch.zeros(vis.shape, dtype=dtype).masked_fill(~vis, torch.finfo(dtype).min)
    else:
        given = torch.zeros(vis.shape).masked_fill(~vis, float("-inf"))
    sc = float(torch.tensor(1 / math.sqrt(D)).to(dtype))
    s_ = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc
    want = torch.softmax(s_.masked_fill(~vis, float("-inf")), -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=given.to(DEV), flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR).cpu()
    assert abi.sdpa_last_kernel() == "tcgen05"
    assert not torch.isnan(got).any()
    assert (got.double() - want).abs().max().item() <= 2e-2
    if kind in ("bool", "additive_min", "additive_f32"):
        # batch element 0 has no padding: its rows equal is_causal=True bit for bit
        ref0 = abi.sdpa_fwd(q[:1].to(DEV), k[:1].to(DEV), v[:1].to(DEV), causal=True, flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR).cpu()
        assert torch.equal(got[:1], ref0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["bool", "bool_odd_address", "additive", "additive_f32_min", "bias"])
@pytest.mark.parametrize("D", [128, 64])
def test_key_padding_masks_on_the_tensor_core_kernel_act_as_sequence_lengths(D, kind, dtype):
    # sequences of different lengths padded to one length, mask [B,1,1,Lk] (bool, additive 0 / -inf, or 0 / the
    # most negative float): a scan finds each batch element's last valid key; its items visit no kv tile past
    # it, and where the valid keys are a prefix the mask is not read again.  Holes stay masked per key; a batch
    # element without any key gives NaN as the reference; an additive row of other values is a bias.
    B, Hq, Hkv, Lq, Lk = 6, 4, 2, 300, 1024
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, D, dtype, seed=81)
    offset = 1 if kind == "bool_odd_address" else 0
    full = torch.zeros(B, 1, 1, Lk + offset, dtype=torch.bool)
    for b, n in enumerate((1024, 513, 17, 0, 700, 128)):
        full[b, :, :, offset:offset + n] = True
    full[4, :, :, offset + 100:offset + 400] = False          # a hole
    vis = full[:, :, :, offset:]
    if kind.startswith("bool"):
        given = full
    elif kind == "additive":
        given = torch.zeros(full.shape).masked_fill(~full, float("-inf")).to(dtype)
    elif kind == "additive_f32_min":
        given = torch.zeros(full.shape).masked_fill(~full, torch.finfo(torch.float32).min)
    else:
        given = (torch.randn(full.shape, generator=torch.Generator().manual_seed(82)) * 2).to(dtype)
    sc = float(torch.tensor(1 / math.sqrt(D)).to(dtype))
    s_ = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc
    s_ = s_ + given[:, :, :, offset:].double() if kind == "bias" else s_.masked_fill(~vis, float("-inf"))
    want = torch.softmax(s_, -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=given.to(DEV)[:, :, :, offset:],
                       flags=abi.SDPA_REF_SCALE | abi.SDPA_FORCE_TENSOR).cpu()
    assert abi.sdpa_last_kernel() == "tcgen05"
    if kind.startswith("bool"):
        ref = O.sdpa(q, k, v, attn_mask=vis, enable_gqa=True)
        assert torch.equal(torch.isnan(got), torch.isnan(ref))
    if kind in ("bool", "bool_odd_address", "additive"):
        assert torch.isnan(got[3]).all()
    fin = ~torch.isnan(want) & ~torch.isnan(got.double())
    assert fin[[0, 1, 2, 4, 5]].all()
    assert (got.double()[fin] - want[fin]).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("kind", ["bool", "additive", "additive_f32_min", "bias"])
def test_decode_kernel_reads_no_keys_past_the_longest_valid_one(kind, offset, dtype):
    # caches of different lengths padded to one length: the kernel finds each batch element's last valid key
    # from the [B,1,1,Lk] mask (bool, or additive 0 / -inf, or 0 / the dtype's most negative value) and shares
    # only that range out among its CTAs; holes inside the range stay masked per key, a batch element without
    # any key gives NaN as in the reference; an additive row with other values ("bias") is applied as given
    B, Hq, Hkv, Lq, Lk = 5, 8, 2, 1, 4096
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, 128, dtype, seed=71)
    full = torch.zeros(B, 1, 1, Lk + 2 * offset, dtype=torch.bool)
    for b, n in enumerate((4096, 2049, 17, 0, 1000)):
        full[b, :, :, 2 * offset:2 * offset + n] = True
    full[4, :, :, 2 * offset + 100:2 * offset + 900] = False          # a hole
    vis = full[:, :, :, 2 * offset:]
    if kind == "bool":
        given, sl = full, slice(2 * offset, None)     # offset 1: the rows start two bytes off a 16-byte boundary
    elif kind == "additive":
        given, sl = torch.zeros(full.shape).masked_fill(~full, float("-inf")).to(dtype), slice(2 * offset, None)
    elif kind == "additive_f32_min":
        given, sl = torch.zeros(full.shape).masked_fill(~full, torch.finfo(torch.float32).min), slice(2 * offset, None)
    else:
        g = torch.Generator().manual_seed(72)
        given, sl = (torch.randn(full.shape, generator=g) * 2).to(dtype), slice(2 * offset, None)
    mask = given[:, :, :, sl]
    sc = float(torch.tensor(1 / math.sqrt(128)).to(dtype))
    s_ = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc
    s_ = s_ + mask.double() if kind == "bias" else s_.masked_fill(~vis, float("-inf"))
    want = torch.softmax(s_, -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=given.to(DEV)[:, :, :, sl], flags=abi.SDPA_REF_SCALE).cpu()
    assert abi.sdpa_last_kernel() == "decode_mma"
    if kind == "bool":
        ref = O.sdpa(q, k, v, attn_mask=mask, enable_gqa=True)
        assert torch.equal(torch.isnan(got), torch.isnan(ref))
    if kind in ("bool", "additive"):
        assert torch.isnan(got[3]).all()                 # no key at all: NaN, as in the reference
    fin = ~torch.isnan(want) & ~torch.isnan(got.double())
    assert fin[[0, 1, 2, 4]].all()
    assert (got.double()[fin] - want[fin]).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["padding", "per_row_bool", "additive", "additive_f32"])
def test_decode_kernel_with_explicit_masks(kind, dtype):
    # batched decoding over caches of different lengths: one or a few query positions, a long cache and a mask;
    # the streaming decode kernel takes these (not the 256-row tensor-core tiles)
    B, Hq, Hkv, Lq, Lk = 3, 8, 2, 2, 1500
    q, k, v = _qkv(B, Hq, Hkv, Lq, Lk, 128, dtype, seed=61)
    g = torch.Generator().manual_seed(62)
    if kind == "padding":
        mask = torch.zeros(B, 1, 1, Lk, dtype=torch.bool)
        for b, n in enumerate((1500, 777, 1)):
            mask[b, :, :, :n] = True
    elif kind == "per_row_bool":
        mask = torch.rand(B, Hq, Lq, Lk, generator=g) > 0.5
        mask[0, 3, 1] = False          # a row without any key: NaN, as in the reference
        mask[..., 0] |= True
        mask[0, 3, 1] = False
    elif kind == "additive":
        mask = (torch.randn(Lq, Lk, generator=g) * 2).to(dtype)
    else:
        mask = torch.randn(B, 1, Lq, Lk, generator=g) * 2
        mask[:, :, :, 900:1000] = float("-inf")
    got = abi.sdpa_fwd(q.to(DEV), k.to(DEV), v.to(DEV), mask=mask.to(DEV), flags=abi.SDPA_REF_SCALE)
    assert abi.sdpa_last_kernel() == "decode_mma"
    if mask.dtype == torch.bool:
        tol_check(got, O.sdpa(q, k, v, attn_mask=mask, enable_gqa=True), f"masked decode {kind} {dtype}")
    else:
        sc = float(torch.tensor(1 / math.sqrt(128)).to(dtype))
        s = (q.double() @ k.double().repeat_interleave(Hq // Hkv, 1).transpose(-1, -2)) * sc + mask.double()
        want = torch.softmax(s, -1) @ v.double().repeat_interleave(Hq // Hkv, 1)
        assert (got.cpu().double() - want).abs().max().item() <= 2e-2, f"masked decode {kind} {dtype}"
