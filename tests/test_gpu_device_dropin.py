"""Drop-in behaviour behind the `paras` device: the same calls a user of the reference makes
(F.scaled_dot_product_attention, torch.ops.aten.rms_norm, torch.ops.torch_paras.swiglu,
torch_paras.nn.*) on device paras:1, compared with CPU PyTorch at the reference's own
tolerance (atol = rtol = 1e-4, dtype and shape must match).  The cases follow the
reference's tests/test_attention_norm_ops.py and tests/test_fused_ops.py one for one."""
import math
import threading

import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O

import torch_paras
from torch_paras import nn as paras_nn

pytestmark = pytest.mark.gpu
DEV = "paras:1"


def assert_close(actual, expected, msg=""):
    actual, expected = actual.cpu(), expected.cpu()
    assert actual.dtype == expected.dtype, f"{msg}: dtype {actual.dtype} vs {expected.dtype}"
    assert actual.shape == expected.shape, f"{msg}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    if actual.dtype.is_floating_point:
        assert torch.allclose(actual, expected, atol=1e-4, rtol=1e-4, equal_nan=True), msg
    else:
        assert torch.equal(actual, expected), msg


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


def _qkv(B=2, H=4, Lq=8, Lk=8, E=16):
    q, k, v = torch.randn(B, H, Lq, E), torch.randn(B, H, Lk, E), torch.randn(B, H, Lk, E)
    return q, k, v, q.to(DEV), k.to(DEV), v.to(DEV)


def test_device_bring_up():
    assert torch_paras.gpu_count() >= 1
    assert torch_paras.device_count() == torch_paras.gpu_count() + 1
    assert torch_paras.is_gpu_device(1)
    assert "B200" in torch_paras.device_name(1) or torch_paras.device_name(1)
    x = torch.randn(64, 64)
    y = x.to(DEV)
    assert y.device.type == "paras" and y.device.index == 1 and y.is_paras
    assert torch.equal(y.cpu(), x)
    assert torch_paras.memory_allocated(1) >= x.numel() * 4
    torch_paras.synchronize()
    torch_paras.synchronize(1)


def test_sdpa_basic():
    q, k, v, dq, dk, dv = _qkv()
    assert_close(F.scaled_dot_product_attention(dq, dk, dv), F.scaled_dot_product_attention(q, k, v))


def test_sdpa_explicit_scale():
    q, k, v, dq, dk, dv = _qkv(E=16)
    s = 1.0 / math.sqrt(32)
    assert_close(F.scaled_dot_product_attention(dq, dk, dv, scale=s),
                 F.scaled_dot_product_attention(q, k, v, scale=s))


def test_sdpa_causal():
    q, k, v, dq, dk, dv = _qkv()
    assert_close(F.scaled_dot_product_attention(dq, dk, dv, is_causal=True),
                 F.scaled_dot_product_attention(q, k, v, is_causal=True))


def test_sdpa_causal_unequal_lengths():
    q, k, v, dq, dk, dv = _qkv(Lq=4, Lk=8)
    assert_close(F.scaled_dot_product_attention(dq, dk, dv, is_causal=True),
                 F.scaled_dot_product_attention(q, k, v, is_causal=True))


def test_sdpa_bool_mask():
    q, k, v, dq, dk, dv = _qkv()
    mask = torch.rand(2, 4, 8, 8) > 0.3
    assert_close(F.scaled_dot_product_attention(dq, dk, dv, attn_mask=mask.to(DEV)),
                 F.scaled_dot_product_attention(q, k, v, attn_mask=mask))


def test_sdpa_additive_mask():
    q, k, v, dq, dk, dv = _qkv()
    bias = torch.randn(2, 4, 8, 8) * 0.1
    assert_close(F.scaled_dot_product_attention(dq, dk, dv, attn_mask=bias.to(DEV)),
                 F.scaled_dot_product_attention(q, k, v, attn_mask=bias))


def test_sdpa_gqa_through_math_op():
    q, k, v = torch.randn(2, 4, 8, 16), torch.randn(2, 2, 8, 16), torch.randn(2, 2, 8, 16)
    ref, _ = torch.ops.aten._scaled_dot_product_attention_math(
        q, k, v, None, 0.0, False, None, scale=None, enable_gqa=True)
    out, _ = torch.ops.aten._scaled_dot_product_attention_math(
        q.to(DEV), k.to(DEV), v.to(DEV), None, 0.0, False, None, scale=None, enable_gqa=True)
    assert_close(out, ref)


def test_sdpa_mismatched_gqa_heads_raises():
    q, k = torch.randn(1, 5, 4, 8).to(DEV), torch.randn(1, 2, 4, 8).to(DEV)
    with pytest.raises(RuntimeError):
        torch.ops.aten._scaled_dot_product_attention_math(q, k, k, None, 0.0, False, None,
                                                          scale=None, enable_gqa=True)


def test_sdpa_bf16_llama_shape_hits_the_tensor_core_kernel():
    g = torch.Generator().manual_seed(1001)
    q = torch.randn(1, 8, 512, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 512, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 512, 128, generator=g).bfloat16()
    out = F.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, enable_gqa=True)
    assert torch_paras._C.sdpa_last_kernel().startswith("tcgen05")
    want = O.sdpa(q, k, v, is_causal=True, enable_gqa=True)
    assert out.dtype == torch.bfloat16 and out.shape == want.shape
    assert (out.cpu().double() - want.double()).abs().max().item() <= 2e-2
    # 3-D input (batch, seq, dim) and a [B, L, H, D] -> transpose(1, 2) view
    q3 = torch.randn(4, 70, 64, generator=g)
    assert_close(F.scaled_dot_product_attention(q3.to(DEV), q3.to(DEV), q3.to(DEV)),
                 F.scaled_dot_product_attention(q3, q3, q3))
    qt = torch.randn(2, 33, 4, 32, generator=g)
    assert_close(F.scaled_dot_product_attention(*(qt.to(DEV).transpose(1, 2),) * 3, is_causal=True),
                 F.scaled_dot_product_attention(*(qt.transpose(1, 2),) * 3, is_causal=True))


def test_sdpa_masks_broadcast_from_the_right_for_3d_and_5d_queries():
    g = torch.Generator().manual_seed(77)
    # 3-D query (batch, seq, dim) with a per-batch mask [B, Lq, Lk]
    q3, k3 = torch.randn(3, 10, 16, generator=g), torch.randn(3, 12, 16, generator=g)
    m3 = torch.rand(3, 10, 12, generator=g) > 0.3
    m3[:, :, 0] = True
    assert_close(F.scaled_dot_product_attention(q3.to(DEV), k3.to(DEV), k3.to(DEV), attn_mask=m3.to(DEV)),
                 F.scaled_dot_product_attention(q3, k3, k3, attn_mask=m3))
    b3 = torch.randn(10, 12, generator=g)                     # shared additive mask
    assert_close(F.scaled_dot_product_attention(q3.to(DEV), k3.to(DEV), k3.to(DEV), attn_mask=b3.to(DEV)),
                 F.scaled_dot_product_attention(q3, k3, k3, attn_mask=b3))
    # 5-D query (a, b, heads, seq, dim) with a mask that broadcasts over some leading dims only
    q5, k5 = torch.randn(2, 3, 2, 6, 8, generator=g), torch.randn(2, 3, 2, 7, 8, generator=g)
    m5 = torch.rand(3, 1, 6, 7, generator=g) > 0.3
    m5[..., 0] = True
    assert_close(F.scaled_dot_product_attention(q5.to(DEV), k5.to(DEV), k5.to(DEV), attn_mask=m5.to(DEV)),
                 F.scaled_dot_product_attention(q5, k5, k5, attn_mask=m5))


def test_sdpa_dropout_draws_the_references_random_stream():
    # F.scaled_dot_product_attention(dropout_p=...) on the device keeps exactly the weights the
    # reference keeps: Philox2x32-10 on (seed, sequence, flat index), the sequence advancing per call
    # as Context::rng_draw does (random_ops.cpp:27-59,140-176, context.cpp:76-83)
    g = torch.Generator().manual_seed(5)
    q, k, v = torch.randn(2, 4, 20, 16, generator=g), torch.randn(2, 4, 33, 16, generator=g), torch.randn(2, 4, 33, 16, generator=g)
    torch_paras.manual_seed(777)
    out1 = F.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), dropout_p=0.3)
    out2 = F.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), dropout_p=0.3)
    want1 = O.sdpa(q, k, v, dropout_p=0.3, rng=(777, 0))
    want2 = O.sdpa(q, k, v, dropout_p=0.3, rng=(777, O.rng_advance(0, 2 * 4 * 20 * 33)))
    assert_close(out1, want1, "dropout, first draw")
    assert_close(out2, want2, "dropout, second draw")
    assert not torch.allclose(out1.cpu(), out2.cpu())
    # the math op returns the weights after dropout; a given dropout_mask replaces the draw
    torch_paras.manual_seed(777)
    o, w = torch.ops.aten._scaled_dot_product_attention_math(q.to(DEV), k.to(DEV), v.to(DEV), None, 0.3, False, None,
                                                             scale=None, enable_gqa=False)
    wo, ww = O.sdpa(q, k, v, dropout_p=0.3, rng=(777, 0), return_weights=True)
    assert_close(o, wo, "math op output")
    assert_close(w, ww, "math op weights")
    assert (w.cpu() == 0).float().mean().item() > 0.2            # about 30 % of the weights were dropped
    dm = (torch.rand(2, 4, 20, 33, generator=g) > 0.5).float()
    o, w = torch.ops.aten._scaled_dot_product_attention_math(q.to(DEV), k.to(DEV), v.to(DEV), None, 0.5, True, dm.to(DEV),
                                                             scale=None, enable_gqa=False)
    wo, ww = O.sdpa(q, k, v, is_causal=True, dropout_p=0.5, dropout_mask=dm, return_weights=True)
    assert_close(o, wo, "dropout_mask output")
    assert_close(w, ww, "dropout_mask weights")
    # bf16, GQA: weights are the reference's own 16-bit values
    qb, kb, vb = q.bfloat16(), k[:, :2].bfloat16(), v[:, :2].bfloat16()
    o, w = torch.ops.aten._scaled_dot_product_attention_math(qb.to(DEV), kb.to(DEV), vb.to(DEV), None, 0.0, True, None,
                                                             scale=None, enable_gqa=True)
    wo, ww = O.sdpa(qb, kb, vb, is_causal=True, enable_gqa=True, return_weights=True)
    assert w.shape == (2, 4, 20, 33) and w.dtype == torch.bfloat16
    assert (w.cpu().float() - ww.float()).abs().max().item() <= 2.0 ** -8     # one bf16 ulp below 1
    assert (o.cpu().float() - wo.float()).abs().max().item() <= 2e-2
    with pytest.raises(RuntimeError, match="too large to materialise"):
        big = torch.empty(1, 64, 4096, 16, dtype=torch.bfloat16).to(DEV)
        torch.ops.aten._scaled_dot_product_attention_math(big, big, big, None, 0.0, True, None, scale=None, enable_gqa=False)


def test_rms_norm_no_weight():
    x = torch.randn(4, 6, 32)
    assert_close(torch.ops.aten.rms_norm(x.to(DEV), [32], None, None),
                 x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6))


def test_rms_norm_with_weight():
    x, w = torch.randn(4, 6, 32), torch.randn(32)
    assert_close(torch.ops.aten.rms_norm(x.to(DEV), [32], w.to(DEV), 1e-5),
                 torch.ops.aten.rms_norm(x, [32], w, 1e-5))
    assert_close(F.rms_norm(x.to(DEV), (32,), w.to(DEV), 1e-5), F.rms_norm(x, (32,), w, 1e-5))


def test_rms_norm_multi_dim_normalized_shape():
    x = torch.randn(3, 4, 5)
    assert_close(torch.ops.aten.rms_norm(x.to(DEV), [4, 5], None, 1e-6),
                 torch.ops.aten.rms_norm(x, [4, 5], None, 1e-6))


def test_rms_norm_shape_mismatch_raises():
    x, w = torch.randn(4, 6, 32).to(DEV), torch.randn(16).to(DEV)
    with pytest.raises(RuntimeError):
        torch.ops.aten.rms_norm(x, [32], w, None)


def test_swiglu_composite_and_manual():
    x, gate = torch.randn(4, 32), torch.randn(4, 32)
    assert_close(torch.ops.torch_paras.swiglu(x.to(DEV), gate.to(DEV)), torch.ops.torch_paras.swiglu(x, gate))
    assert_close(torch.ops.torch_paras.swiglu(x.to(DEV), gate.to(DEV)), x * F.silu(gate))
    # broadcasting, as the composite allows
    assert_close(torch.ops.torch_paras.swiglu(x.to(DEV), gate[:1].to(DEV)), x * F.silu(gate[:1]))


def test_fused_rms_norm_forward_backward():
    x, w = torch.randn(4, 8, requires_grad=True), torch.randn(8, requires_grad=True)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    ref.sum().backward()
    xd = x.detach().to(DEV).requires_grad_()
    wd = w.detach().to(DEV).requires_grad_()
    out = paras_nn.rms_norm(xd, wd, 1e-6)
    assert_close(out.detach(), ref.detach())
    out.sum().backward()
    assert_close(xd.grad, x.grad)
    assert_close(wd.grad, w.grad)


def test_fused_swiglu_forward_backward():
    gate, up = torch.randn(4, 8, requires_grad=True), torch.randn(4, 8, requires_grad=True)
    ref = F.silu(gate) * up
    ref.sum().backward()
    gd = gate.detach().to(DEV).requires_grad_()
    ud = up.detach().to(DEV).requires_grad_()
    out = paras_nn.swiglu(gd, ud)
    assert_close(out.detach(), ref.detach())
    out.sum().backward()
    assert_close(gd.grad, gate.grad)
    assert_close(ud.grad, up.grad)


def test_rotate_half_forward_backward():
    x = torch.randn(4, 8, requires_grad=True)
    x1, x2 = x.chunk(2, dim=-1)
    ref = torch.cat((-x2, x1), dim=-1)
    ref.sum().backward()
    xd = x.detach().to(DEV).requires_grad_()
    out = paras_nn.rotate_half(xd)
    assert_close(out.detach(), ref.detach())
    out.sum().backward()
    assert_close(xd.grad, x.grad)


def test_copy_cases():
    a, src = torch.randn(4, 5), torch.randn(4, 5)
    assert_close(a.to(DEV).clone().copy_(src.to(DEV)), a.clone().copy_(src))
    with pytest.raises(RuntimeError):
        a.to(DEV).clone().copy_(torch.randn(5).to(DEV))          # broadcasting copy is refused
    h = torch.randn(4, 5).half()
    assert_close(a.to(DEV).clone().copy_(h.to(DEV)), a.clone().copy_(h))   # dtype cast on device
    d = torch.randn(4, 5).to(DEV)
    d.copy_(src)
    assert_close(d, src)
    t = torch.randn(6, 7)
    assert_close(t.to(DEV).t().contiguous(), t.t().contiguous())            # strided device copy
    assert_close(t.to(DEV)[1:5, ::2], t[1:5, ::2])
    big = torch.randn(3000, 3000)                                            # several staging chunks
    assert_close(big.to(DEV), big)
    assert torch.zeros(5, device=DEV).cpu().abs().sum().item() == 0
    assert torch.full((3,), 7.0, device=DEV).cpu().tolist() == [7.0, 7.0, 7.0]
    one = torch.tensor([1.5, -2.25, 3.0])
    assert one.to(DEV)[1].item() == -2.25                                     # _local_scalar_dense


def test_paras_memory_viewed_as_cuda_tensor():
    from torch_paras import sharding
    x = torch.randn(33, 65).bfloat16()
    d = x.to(DEV)
    torch_paras.synchronize(1)
    c = sharding.as_cuda(d)
    assert c.device.type == "cuda" and c.dtype == torch.bfloat16 and c.shape == d.shape
    assert torch.equal(c.cpu(), x)
    c.mul_(2)                       # same memory: the paras tensor sees the change
    torch.cuda.synchronize()
    assert torch.equal(d.cpu(), x * 2)


def test_concurrent_dispatch_from_python_threads():
    x = torch.randn(256, 512)
    want = F.silu(x) * x
    errs = []

    def work():
        try:
            for _ in range(20):
                d = x.to(DEV)
                assert torch.allclose(torch.ops.paras.swiglu(d, d).cpu(), want, atol=1e-4, rtol=1e-4)
        except Exception as e:  # noqa: BLE001
            errs.append(e)

    ts = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs, errs[0]


def test_attention_host_streams_batches_through_the_gpu():
    # host operands in, host result out, in one call; pinned and pageable, GQA, causal and not
    g = torch.Generator().manual_seed(3)
    for (B, Hq, Hkv, L, causal, dtype) in [(5, 4, 2, 384, True, torch.bfloat16),
                                           (3, 2, 2, 200, False, torch.float16),
                                           (2, 2, 1, 64, True, torch.float32)]:
        q = torch.randn(B, Hq, L, 128, generator=g).to(dtype)
        k = torch.randn(B, Hkv, L, 128, generator=g).to(dtype)
        v = torch.randn(B, Hkv, L, 128, generator=g).to(dtype)
        want = O.sdpa(q, k, v, is_causal=causal, enable_gqa=Hq != Hkv)
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        got = paras_nn.attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), is_causal=causal)
        assert got.device.type == "cpu" and got.is_pinned() and got.dtype == dtype
        assert (got.double() - want.double()).abs().max().item() <= tol
        out = torch.empty_like(q)  # pageable operands and result
        got2 = paras_nn.attention_host(q, k, v, is_causal=causal, out=out)
        assert got2 is out and torch.equal(out, got)
    with pytest.raises(RuntimeError):
        paras_nn.attention_host(q, k, v, device=0)


def test_memory_limit_makes_allocation_fail_like_a_full_device():
    # out-of-memory handling without exhausting a GPU: a host-side cap on the pool
    import torch_paras
    torch_paras.synchronize()
    base = torch_paras.memory_allocated(1)
    torch_paras.set_memory_limit(base + (64 << 20), 1)
    try:
        small = torch.empty(32 << 20, dtype=torch.uint8, device="paras:1")
        with pytest.raises(RuntimeError, match="out of memory"):
            torch.empty(128 << 20, dtype=torch.uint8, device="paras:1")
        del small
        # an operator that needs scratch fails the same way and leaves the device usable
        q = torch.randn(1, 2, 64, 64, device="paras:1")
        torch_paras.set_memory_limit(torch_paras.memory_allocated(1) + 1024, 1)
        with pytest.raises(RuntimeError, match="out of memory"):
            torch.empty(1 << 20, dtype=torch.uint8, device="paras:1")
    finally:
        torch_paras.set_memory_limit(0, 1)
    out = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.cpu(), q.cpu(), q.cpu(), is_causal=True)
    assert torch.allclose(out.cpu(), ref, atol=1e-4, rtol=1e-4)


def test_copies_casts_and_transposes_match_cpu_for_every_layout():
    # the copy kernels behind .contiguous() / .to(dtype) / copy_: rows with a contiguous last dimension,
    # transposes of the last two dimensions, general permutations and slices, every element type
    import itertools
    g = torch.Generator().manual_seed(0)

    def same(name, fn):
        want = fn(lambda t: t)
        got = fn(lambda t: t.to("paras:1")).cpu()
        assert got.shape == want.shape and got.dtype == want.dtype and torch.equal(got, want), name

    for dt in (torch.bfloat16, torch.float16, torch.float32, torch.int32, torch.int16, torch.float64):
        x = (torch.randn(3, 40, 8, 64, generator=g) * 50).to(dt)
        same(f"transpose(1,2) {dt}", lambda dev: dev(x).transpose(1, 2).contiguous())
        same(f"transpose(-1,-2) {dt}", lambda dev: dev(x).transpose(-1, -2).contiguous())
        same(f"permute {dt}", lambda dev: dev(x).permute(3, 0, 2, 1).contiguous())
        same(f"slice {dt}", lambda dev: dev(x)[:, 3:37, :, 8:56].contiguous())
        same(f"clone {dt}", lambda dev: dev(x).clone())
        y = (torch.randn(333, 517, generator=g) * 9).to(dt)
        same(f"t() {dt}", lambda dev: dev(y).t().contiguous())
        same(f"t() of a slice {dt}", lambda dev: dev(y)[5:300, 7:500].t().contiguous())
    for a, b in itertools.permutations((torch.bfloat16, torch.float16, torch.float32), 2):
        x = (torch.randn(5, 33, 128, generator=g) * 3).to(a)
        same(f"cast {a} -> {b}", lambda dev: dev(x).to(b))
        same(f"cast of a view {a} -> {b}", lambda dev: dev(x).transpose(0, 1).to(b))
        z = torch.randn(1000003, generator=g).to(a)
        same(f"cast, odd length {a} -> {b}", lambda dev: dev(z).to(b))
        z2 = torch.randn(8 * 4097, generator=g).to(a)
        same(f"cast, 8 x 4097 {a} -> {b}", lambda dev: dev(z2).to(b))
    dst = torch.zeros(4, 64, 16, 128).bfloat16()
    src = torch.randn(4, 16, 64, 128, generator=g).bfloat16()
    d1 = dst.clone()
    d1.transpose(1, 2).copy_(src)
    d2 = dst.clone().to("paras:1")
    d2.transpose(1, 2).copy_(src.to("paras:1"))
    assert torch.equal(d1, d2.cpu())
