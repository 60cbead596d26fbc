"""The allocation-free attention entry point (paras_b200_sdpa_fwd_static_scratch).

It exists for callers that cannot allocate device memory at call time -- e.g. a serving
process that handed the whole GPU to its own memory manager at start-up, or a decode loop
with no latency budget for an allocator call.  Its split-KV scratch is a fixed array inside
the library, so the checks here are: same result as the regular entry point and as the CPU
oracle, twice in a row (the array is shared between calls and keeps the previous call's
contents), and a clear refusal when a problem's partial results do not fit the array.
"""
import ctypes

import pytest
import torch

import torch_paras  # noqa: F401
from torch_paras import abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _decode_inputs(dtype, seed, B=2, Hq=8, Hkv=2, Lk=4096, D=128):
    g = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, device=DEV).to(dtype)  # noqa: E731
    return mk(B, Hq, 1, D), mk(B, Hkv, Lk, D), mk(B, Hkv, Lk, D)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
def test_static_scratch_matches_regular_entry_point_twice(dtype, tol):
    outs = []
    for call in range(2):                       # second call reuses the array the first one left dirty
        q, k, v = _decode_inputs(dtype, seed=100 + call)
        out = torch.empty_like(q)               # the caller owns inputs and outputs
        abi.sdpa_fwd_static_scratch(q, k, v, out=out, flags=abi.SDPA_REF_SCALE)
        assert abi.sdpa_last_kernel() == "simt_splitkv_static"   # the scratch really was used
        want = abi.sdpa_fwd(q, k, v, flags=abi.SDPA_REF_SCALE)
        err = (out.float() - want.float()).abs().max().item()
        assert err <= tol, f"call {call}: max-abs {err} > {tol} against the regular entry point"
        # for fp32 the regular entry point runs the same kernel (with pool scratch), so the
        # independent expectation is the oracle: the reference's arithmetic on the host
        gold = O.sdpa(q.cpu(), k.cpu(), v.cpu(), enable_gqa=True)
        err = (out.cpu().double() - gold.double()).abs().max().item()
        assert err <= tol, f"call {call}: max-abs {err} > {tol} against the oracle"
        assert torch.isfinite(out.float()).all()
        outs.append(out)
    assert not torch.equal(outs[0], outs[1])    # different inputs gave different results


def test_static_scratch_causal_prefill_shape_needs_no_scratch():
    g = torch.Generator(device=DEV).manual_seed(7)
    q = torch.randn(1, 2, 64, 64, generator=g, device=DEV)
    out = abi.sdpa_fwd_static_scratch(q, q, q, causal=True)
    want = abi.sdpa_fwd(q, q, q, causal=True)
    assert (out - want).abs().max().item() <= 1e-4
    gold = O.sdpa(q.cpu(), q.cpu(), q.cpu(), is_causal=True)
    assert (out.cpu() - gold).abs().max().item() <= 1e-4


def test_static_scratch_rejects_what_does_not_fit():
    cap = abi.lib().paras_b200_sdpa_static_scratch_bytes()
    assert cap == 4 << 20
    # 2048 query rows x 3 splits x 256 fp32 partials = 6.3 MB: more than the array holds
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn(8, 64, 4, 256, generator=g, device=DEV).bfloat16()
    k = torch.randn(8, 8, 1024, 256, generator=g, device=DEV).bfloat16()
    assert abi.sdpa_workspace_bytes(q, k, k, flags=abi.SDPA_FORCE_SIMT) > cap
    with pytest.raises(RuntimeError, match="static scratch holds"):
        abi.sdpa_fwd_static_scratch(q, k, k)
    abi.sdpa_fwd(q, k, k)        # the regular entry point takes the same problem
    a = abi.SdpaArgs()
    a.dtype, a.B, a.Hq, a.Hkv, a.Lq, a.Lk, a.D = abi.BF16, 1, 5, 2, 1, 16, 128
    assert abi.lib().paras_b200_sdpa_fwd_static_scratch(ctypes.byref(a)) == -1
