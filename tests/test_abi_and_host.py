"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares,
reports errors instead of computing without a GPU, and the host side of the `paras` device
(paras:0 tensors, copies, error behaviour of the operator layer) works."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

import torch_paras
from torch_paras import abi

HEADER = os.path.join(ROOT, "include", "paras_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(paras_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = abi.lib()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/paras_b200.h but not exported"
    assert sorted(abi.EXPORTS) == names


def test_abi_version_and_backend_name():
    lib = abi.lib()
    assert lib.paras_b200_abi_version() == 2
    assert lib.paras_b200_backend_name().decode().startswith("paras-b200")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU error path")
def test_compute_entry_points_fail_loudly_without_gpu():
    lib = abi.lib()
    assert lib.paras_b200_device_count() == 0
    buf = (ctypes.c_char * 64)()
    st = lib.paras_b200_swiglu_fwd(0, buf, buf, buf, 16, abi.BF16, abi.ROUND_ONCE, None)
    assert st == -4  # PARAS_E_NODEVICE
    assert b"no CUDA GPU" in lib.paras_b200_last_error()
    st = lib.paras_b200_rmsnorm_fwd(0, buf, buf, buf, None, 1, 16, 1e-6, abi.BF16, 0, None)
    assert st == -4
    a = abi.SdpaArgs()
    a.dtype, a.B, a.Hq, a.Hkv, a.Lq, a.Lk, a.D = abi.BF16, 1, 1, 1, 1, 1, 128
    assert lib.paras_b200_sdpa_fwd(ctypes.byref(a)) == -4
    p = ctypes.c_void_p()
    assert lib.paras_b200_malloc_async(0, 64, None, ctypes.byref(p)) == -4


def test_argument_validation_comes_before_device_use():
    lib = abi.lib()
    a = abi.SdpaArgs()
    a.dtype, a.B, a.Hq, a.Hkv, a.Lq, a.Lk, a.D = abi.BF16, 1, 5, 2, 4, 4, 8
    assert lib.paras_b200_sdpa_fwd(ctypes.byref(a)) == -1  # heads do not divide
    assert b"multiple of key/value heads" in lib.paras_b200_last_error()
    a.Hq = 4
    a.dtype = 7
    assert lib.paras_b200_sdpa_fwd(ctypes.byref(a)) == -2
    assert lib.paras_b200_sdpa_fwd(None) == -1
    buf = (ctypes.c_char * 64)()
    assert lib.paras_b200_swiglu_fwd(0, buf, buf, buf, -1, abi.BF16, 0, None) == -1
    assert lib.paras_b200_rotate_half(0, buf, buf, 1, 3, abi.F32, 0, None) == -1


def test_split_kv_scratch_parts_are_aligned_for_every_shape():
    # the {max, sum} pairs are read and written as 8-byte float2, the partial outputs as fp32;
    # odd head dims with odd split counts must not push either part off its alignment
    for rows in (1, 2, 3, 5, 7, 63, 64, 1000, 4097):
        for D in (1, 3, 63, 64, 65, 127, 128, 255, 256):
            for splits in (2, 3, 5, 7, 8, 33):
                ml, o, n = abi.sdpa_split_layout(rows, D, splits)
                assert ml % 16 == 0 and o % 16 == 0, (rows, D, splits, ml, o)
                assert o >= ml + 8 * rows * splits            # the parts do not overlap
                assert n >= o + 4 * rows * splits * D         # and the total covers both
    assert abi.sdpa_split_layout(5, 63, 1) == (0, 0, 0)       # one split needs no scratch


def test_device_numbering_and_host_device():
    assert torch_paras.device_count() == 1 + torch_paras.gpu_count()
    assert torch_paras.device_name(0) == "host"
    assert not torch_paras.is_gpu_device(0)
    assert torch_paras.is_available()
    assert not torch.paras.is_bad_fork()
    with pytest.raises(RuntimeError):
        torch_paras.device_name(torch_paras.device_count())


def test_host_tensor_round_trip_views_and_fill():
    x = torch.randn(4, 5)
    y = x.to("paras:0")
    assert y.device.type == "paras" and y.device.index == 0
    assert torch.equal(y.cpu(), x)
    assert torch.equal(y.t().contiguous().cpu(), x.t().contiguous())
    assert torch.equal(y.view(20).cpu(), x.view(20))
    assert torch.equal(y[1:3, ::2].cpu(), x[1:3, ::2])
    z = torch.zeros(3, 2, device="paras:0")
    assert torch.equal(z.cpu(), torch.zeros(3, 2))
    z.fill_(2.5)
    assert torch.equal(z.cpu(), torch.full((3, 2), 2.5))
    assert y.sum().item() == pytest.approx(x.sum().item(), rel=1e-6)   # boxed CPU fallback
    assert torch.equal(y.half().cpu(), x.half())
    h = torch.empty(0, device="paras:0")
    assert h.numel() == 0
    with pytest.raises(RuntimeError):
        y.copy_(torch.randn(3, 3).to("paras:0"))   # element count mismatch


def test_hot_path_ops_refuse_the_host_device():
    q = torch.randn(1, 2, 4, 8).to("paras:0")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        torch.nn.functional.scaled_dot_product_attention(q, q, q)
    x = torch.randn(4, 8).to("paras:0")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        torch.ops.paras.swiglu(x, x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        torch.ops.aten.rms_norm(x, [8], None, None)


def test_operator_argument_errors_match_the_reference():
    # checked before any device work, so they can be exercised on the host device
    x = torch.randn(4, 6, 32).to("paras:0")
    w = torch.randn(16).to("paras:0")
    with pytest.raises(RuntimeError, match="weight shape must equal normalized_shape"):
        torch.ops.aten.rms_norm(x, [32], w, None)
    with pytest.raises(RuntimeError, match="normalized_shape does not match"):
        torch.ops.aten.rms_norm(x, [31], None, None)
    q = torch.randn(1, 5, 4, 8).to("paras:0")
    k = torch.randn(1, 2, 4, 8).to("paras:0")
    with pytest.raises(RuntimeError):
        torch.ops.aten._scaled_dot_product_attention_math(q, k, k, None, 0.0, False, None,
                                                          scale=None, enable_gqa=True)
    with pytest.raises(RuntimeError, match="mutually exclusive"):
        torch.nn.functional.scaled_dot_product_attention(
            k, k, k, attn_mask=torch.ones(4, 4, dtype=torch.bool).to("paras:0"), is_causal=True)
    with pytest.raises(RuntimeError, match="same shape"):
        torch.ops.paras.swiglu(torch.randn(4, 8).to("paras:0"), torch.randn(4, 4).to("paras:0"))
    with pytest.raises(RuntimeError, match="must be even"):
        torch.ops.paras.rotate_half(torch.randn(4, 7).to("paras:0"))


def test_torch_paras_swiglu_has_a_cpu_kernel():
    # the reference registers torch_paras::swiglu for CPU tensors too (rms_swiglu_ops.cpp:108-110)
    x, g = torch.randn(4, 32), torch.randn(4, 32)
    assert torch.allclose(torch.ops.torch_paras.swiglu(x, g), x * torch.nn.functional.silu(g))
