"""The projections either side of the path: the tcgen05 GEMM behind paras_b200_gemm, called
through the C ABI and through the `paras` device (aten::mm / bmm / addmm / linear and
paras::swiglu_linear), against what the reference computes for them: libtorch's CPU GEMM on
host copies (csrc/ops/vision_ops.cpp:248-309, 388-423).

Tolerance: both sides accumulate in fp32 and round once, but not in the same order, so a
result may land on the neighbouring 16-bit value: |got - want| <= 2^-7 |want| + 2e-2 for bf16
(2^-10 |want| + 2e-2 for fp16), and at least 99 % of the elements must be bit-equal.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O

import torch_paras
from torch_paras import abi, nn as paras_nn

pytestmark = pytest.mark.gpu
CUDA = "cuda:0"
DEV = "paras:1"


def close16(got, want, name, exact_share=0.99):
    got = got.detach().cpu()
    assert got.dtype == want.dtype and got.shape == want.shape, name
    g, w = got.double(), want.double()
    rel = 2.0 ** -7 if want.dtype == torch.bfloat16 else 2.0 ** -10
    bad = (g - w).abs() > rel * w.abs() + 2e-2
    assert not bad.any(), f"{name}: {int(bad.sum())} elements off, worst {(g - w).abs().max():.3e}"
    if want.numel():
        share = (got == want).double().mean().item()
        assert share >= exact_share, f"{name}: only {share:.4f} of the elements are bit-equal"


def rand(shape, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


SHAPES = [(128, 256, 64), (256, 512, 512), (300, 520, 136), (1, 8, 8), (77, 1000, 264),
          (640, 384, 1000), (129, 257 * 8, 72),
          (1000, 128, 520), (333, 72, 264), (4096, 128, 2048)]   # N <= 128: half-width tiles


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_abi_against_host_gemm(shape, dtype):
    M, N, K = shape
    a, w, b = rand((M, K), 1, dtype), rand((N, K), 2, dtype), rand((K, N), 3, dtype)
    bias = rand((N,), 4, dtype)
    close16(abi.gemm(a.to(CUDA), w.to(CUDA)), O.linear(a, w), f"A W^T {shape}")
    close16(abi.gemm(a.to(CUDA), b.to(CUDA), b_layout=abi.GEMM_B_KN), O.mm(a, b), f"A B {shape}")
    close16(abi.gemm(a.to(CUDA), w.to(CUDA), bias=bias.to(CUDA)), O.linear(a, w, bias), f"bias {shape}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(256, 256, 128), (500, 1000, 264), (64, 136, 2048)])
def test_swiglu_epilogue_against_two_linears_and_swiglu(shape, dtype):
    M, Fd, K = shape
    x, wg, wu = rand((M, K), 1, dtype), rand((Fd, K), 2, dtype, 0.05), rand((Fd, K), 3, dtype, 0.05)
    got = abi.gemm(x.to(CUDA), wg.to(CUDA), up_weight=wu.to(CUDA))
    # a neighbouring 16-bit value of either projection moves the product, so fewer exact hits
    close16(got, O.swiglu_linear(x, wg, wu), f"swiglu epilogue {shape}", exact_share=0.97)


def test_batched_and_strided_operands():
    dtype = torch.bfloat16
    a, b = rand((6, 200, 136), 1, dtype), rand((6, 136, 328), 2, dtype)
    close16(abi.gemm(a.to(CUDA), b.to(CUDA), b_layout=abi.GEMM_B_KN), O.bmm(a, b), "bmm")
    # rows that are slices of a wider matrix (leading dimension > row length)
    wide = rand((300, 512), 3, dtype)
    w = rand((264, 256), 4, dtype)
    close16(abi.gemm(wide.to(CUDA)[:, 128:384], w.to(CUDA)), O.linear(wide[:, 128:384], w), "strided A")
    out = torch.zeros(300, 512, dtype=dtype, device=CUDA)
    abi.gemm(wide.to(CUDA)[:, 128:384], w.to(CUDA), out=out[:, 8:272])
    close16(out[:, 8:272], O.linear(wide[:, 128:384], w), "strided C")
    assert float(out[:, :8].abs().sum()) == 0.0 and float(out[:, 272:].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 4096, 4096), (16, 1024, 2048), (1, 520, 1024), (512, 1032, 3584),
                                   (130, 128, 4096), (8, 72, 8192), (200, 264, 1536)])
def test_few_tiles_and_a_long_k_split_the_k_range(shape, dtype):
    # The projections of a decode step (M = the batch): too few output tiles to fill the GPU, so the
    # K range runs as slices whose fp32 partial sums a second kernel adds up.  Same tolerance: one
    # rounding at the end, on either side; with K this long and outputs this few, a handful of results on
    # the neighbouring 16-bit value already is more than 1 % of them, hence the lower exact share.
    M, N, K = shape
    a, w, b = rand((M, K), 1, dtype, 0.5), rand((N, K), 2, dtype, 0.5), rand((K, N), 3, dtype, 0.5)
    bias = rand((N,), 4, dtype)
    close16(abi.gemm(a.to(CUDA), w.to(CUDA)), O.linear(a, w), f"A W^T {shape}", exact_share=0.97)
    close16(abi.gemm(a.to(CUDA), b.to(CUDA), b_layout=abi.GEMM_B_KN), O.mm(a, b), f"A B {shape}", exact_share=0.97)
    close16(abi.gemm(a.to(CUDA), w.to(CUDA), bias=bias.to(CUDA)), O.linear(a, w, bias), f"bias {shape}", exact_share=0.97)
    # into a slice of a wider matrix: the columns either side stay untouched
    out = torch.zeros(M, N + 16, dtype=dtype, device=CUDA)
    abi.gemm(a.to(CUDA), w.to(CUDA), out=out[:, 8:N + 8])
    close16(out[:, 8:N + 8], O.linear(a, w), f"strided C {shape}", exact_share=0.97)
    assert float(out[:, :8].abs().sum()) == 0.0 and float(out[:, N + 8:].abs().sum()) == 0.0
    # the same call twice gives the same bits (slices are summed in a fixed order)
    x, y = abi.gemm(a.to(CUDA), w.to(CUDA)), abi.gemm(a.to(CUDA), w.to(CUDA))
    assert torch.equal(x, y)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2304, 2304, 520), (2400, 2056, 264), (5000, 1032, 256), (1290, 4360, 1096)])
def test_large_projections_on_cta_pairs(shape, dtype):
    # At least half a wave of 256 x 256 tiles: the kernel that computes a tile on two CTAs of a cluster.
    # Ragged M, N and K against the same host GEMM, with and without bias, and the same call on the
    # single-CTA kernel must give the same bits (both accumulate a tile's K range in one fp32 chain).
    M, N, K = shape
    a, w = rand((M, K), 1, dtype, 0.5), rand((N, K), 2, dtype, 0.5)
    bias = rand((N,), 4, dtype)
    ad, wd = a.to(CUDA), w.to(CUDA)
    got = abi.gemm(ad, wd)
    close16(got, O.linear(a, w), f"pair A W^T {shape}")
    close16(abi.gemm(ad, wd, bias=bias.to(CUDA)), O.linear(a, w, bias), f"pair bias {shape}")
    out = torch.zeros(M, N + 16, dtype=dtype, device=CUDA)
    abi.gemm(ad, wd, out=out[:, 8:N + 8])
    assert torch.equal(out[:, 8:N + 8], got)
    assert float(out[:, :8].abs().sum()) == 0.0 and float(out[:, N + 8:].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (7, 520, 1000), (16, 128, 256), (33, 6144, 4096), (64, 4096, 1096),
                                   (100, 1032, 8192), (128, 2056, 4096), (48, 28672, 512), (5, 4096, 14336),
                                   (130, 4096, 1024), (200, 19000, 264), (256, 6144, 4096)])
def test_decode_step_projections_on_the_weight_streaming_kernel(shape, dtype):
    # At most 128 rows against a weight: the weight rows sit on the MMA's M side, K is split inside a
    # cluster and summed through distributed shared memory in a fixed order (the same bits every run).
    M, N, K = shape
    a, w = rand((M, K), 1, dtype, 0.5), rand((N, K), 2, dtype, 0.5)
    bias = rand((N,), 4, dtype)
    ad, wd = a.to(CUDA), w.to(CUDA)
    got = abi.gemm(ad, wd)
    close16(got, O.linear(a, w), f"skinny A W^T {shape}", exact_share=0.97)
    close16(abi.gemm(ad, wd, bias=bias.to(CUDA)), O.linear(a, w, bias), f"skinny bias {shape}", exact_share=0.97)
    assert torch.equal(abi.gemm(ad, wd), got)
    out = torch.zeros(M, N + 16, dtype=dtype, device=CUDA)
    abi.gemm(ad, wd, out=out[:, 8:N + 8])
    assert torch.equal(out[:, 8:N + 8], got)
    assert float(out[:, :8].abs().sum()) == 0.0 and float(out[:, N + 8:].abs().sum()) == 0.0
    # rows that are slices of a wider activation matrix
    wide = rand((M, K + 64), 9, dtype, 0.5)
    close16(abi.gemm(wide.to(CUDA)[:, 32:K + 32], wd), O.linear(wide[:, 32:K + 32], w), f"skinny strided A {shape}",
            exact_share=0.97)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1024, 512), (16, 14336, 4096), (64, 1704, 1000), (100, 2056, 1096), (128, 520, 264)])
def test_decode_step_gate_up_projection_with_swiglu(shape, dtype):
    # paras::swiglu_linear with a handful of rows: 64 gate-weight rows over 64 up-weight rows per block
    M, Fd, K = shape
    x, wg, wu = rand((M, K), 1, dtype), rand((Fd, K), 2, dtype, 0.05), rand((Fd, K), 3, dtype, 0.05)
    got = abi.gemm(x.to(CUDA), wg.to(CUDA), up_weight=wu.to(CUDA))
    want = O.swiglu_linear(x, wg, wu)
    # Either projection may land on the neighbouring 16-bit value (K = 4096 terms summed in another order),
    # which moves silu(g) * u by up to an ulp before its own rounding: two ulps of the result, not one.
    g, w = got.cpu().double(), want.double()
    ulp2 = 2.0 ** -6 if dtype == torch.bfloat16 else 2.0 ** -9
    bad = (g - w).abs() > ulp2 * w.abs() + 2e-2
    assert not bad.any(), f"skinny swiglu {shape}: {int(bad.sum())} elements off, worst {(g - w).abs().max():.3e}"
    # (with K = 4096 each projection differs from the host GEMM's rounding in 1-1.5 % of its elements)
    assert (got.cpu() == want).double().mean().item() >= 0.95
    assert torch.equal(abi.gemm(x.to(CUDA), wg.to(CUDA), up_weight=wu.to(CUDA)), got)


@pytest.mark.parametrize("shape", [(2304, 2304, 520), (1296, 4360, 264)])
def test_transposed_operands_and_batches_on_cta_pairs(shape):
    # the gradients of a linear layer: dX = dY W (B as [K, N] rows), dW = dY^T X (A as [K, M] rows), and bmm
    M, N, K = shape
    dtype = torch.bfloat16
    a, at, w, b = rand((M, K), 1, dtype, 0.5), rand((K, M), 5, dtype, 0.5), rand((N, K), 2, dtype, 0.5), rand((K, N), 3, dtype, 0.5)
    bias = rand((N,), 4, dtype)
    close16(abi.gemm(a.to(CUDA), b.to(CUDA), b_layout=abi.GEMM_B_KN), O.mm(a, b), f"pair A B {shape}")
    close16(abi.gemm(a.to(CUDA), b.to(CUDA), b_layout=abi.GEMM_B_KN, bias=bias.to(CUDA)), O.linear(a, b.t().contiguous(), bias),
            f"pair A B + bias {shape}")
    close16(abi.gemm(at.to(CUDA), w.to(CUDA), a_transposed=True), O.mm(at.t(), w.t()), f"pair A^T W^T {shape}")
    close16(abi.gemm(at.to(CUDA), b.to(CUDA), a_transposed=True, b_layout=abi.GEMM_B_KN), O.mm(at.t(), b), f"pair A^T B {shape}")
    x3, y3 = rand((3, 1300, 520), 6, dtype, 0.5), rand((3, 520, 1800), 7, dtype, 0.5)
    close16(abi.gemm(x3.to(CUDA), y3.to(CUDA), b_layout=abi.GEMM_B_KN), O.bmm(x3, y3), "pair bmm")
    w3 = rand((3, 1800, 520), 8, dtype, 0.5)
    close16(abi.gemm(x3.to(CUDA), w3.to(CUDA)), O.bmm(x3, w3.transpose(1, 2)), "pair batched A W^T")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_and_row_scale_epilogues_on_cta_pairs(dtype):
    M, Fd, K = 1300, 1704, 512
    x, wg, wu = rand((M, K), 1, dtype), rand((Fd, K), 2, dtype, 0.05), rand((Fd, K), 3, dtype, 0.05)
    got = abi.gemm(x.to(CUDA), wg.to(CUDA), up_weight=wu.to(CUDA))
    close16(got, O.swiglu_linear(x, wg, wu), "pair swiglu epilogue", exact_share=0.97)
    M, N, K = 2304, 2304, 512
    x = rand((M, K), 11, dtype, 1.5)
    wn = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(12))).to(dtype)
    w = rand((N, K), 13, dtype, 0.05)
    y, _ = O.rms_norm_fused(x, wn, 1e-6)
    want = O.linear(y, w).double()
    got = abi.rms_norm_linear(x.to(CUDA), wn.to(CUDA), w.to(CUDA), 1e-6).cpu().double()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    err = (got - want).abs()
    assert (err <= 2 * ulp * want.abs() + 2e-2 * want.abs().max().item()).all(), f"worst {err.max().item():.3e}"


@pytest.mark.parametrize("shape", [(128, 256, 64), (304, 520, 136), (1000, 264, 392), (520, 128, 1000), (304, 64, 136)])
def test_transposed_a_operand(shape):
    # A given as [K, M] (rows of M): C = A^T B, with B in either layout
    M, N, K = shape
    dtype = torch.bfloat16
    at, w, b = rand((K, M), 1, dtype), rand((N, K), 2, dtype), rand((K, N), 3, dtype)
    close16(abi.gemm(at.to(CUDA), w.to(CUDA), a_transposed=True), O.mm(at.t(), w.t()), f"A^T W^T {shape}")
    close16(abi.gemm(at.to(CUDA), b.to(CUDA), a_transposed=True, b_layout=abi.GEMM_B_KN),
            O.mm(at.t(), b), f"A^T B {shape}")


def test_operands_the_kernel_does_not_take_are_refused():
    a = torch.randn(64, 64, device=CUDA)
    with pytest.raises(RuntimeError):
        abi.gemm(a, a)                                   # fp32
    h = torch.randn(64, 68, device=CUDA).bfloat16()
    with pytest.raises(RuntimeError):
        abi.gemm(h[:, :60], h[:, :60])                   # leading dimension not a multiple of 8
    z = abi.gemm(torch.empty(0, 64, device=CUDA).bfloat16(), torch.empty(32, 64, device=CUDA).bfloat16())
    assert z.shape == (0, 32)


def test_device_ops_route_to_the_kernel_and_fall_back_like_the_reference():
    dtype = torch.bfloat16
    x, w, bias = rand((4, 50, 256), 1, dtype), rand((384, 256), 2, dtype), rand((384,), 3, dtype)
    dx, dw, db = x.to(DEV), w.to(DEV), bias.to(DEV)
    close16(F.linear(dx, dw, db), O.linear(x, w, bias), "F.linear")
    close16(F.linear(dx, dw), O.linear(x, w), "F.linear no bias")
    a, b = rand((200, 256), 4, dtype), rand((256, 136), 5, dtype)
    close16(torch.mm(a.to(DEV), b.to(DEV)), O.mm(a, b), "mm")
    close16(a.to(DEV) @ w.to(DEV).t(), O.mm(a, w.t()), "x @ w.t()")
    c = rand((136,), 6, dtype)
    close16(torch.addmm(c.to(DEV), a.to(DEV), b.to(DEV)), O.addmm(c, a, b), "addmm")
    a3, b3 = rand((3, 64, 72), 7, dtype), rand((3, 72, 40), 8, dtype)
    close16(torch.bmm(a3.to(DEV), b3.to(DEV)), O.bmm(a3, b3), "bmm")
    # fp32 and odd shapes keep the reference's host route: results are libtorch's, exactly
    a32, b32 = torch.randn(33, 17), torch.randn(17, 5)
    assert torch.equal(torch.mm(a32.to(DEV), b32.to(DEV)).cpu(), torch.mm(a32, b32))
    odd_a, odd_b = rand((9, 13), 9, dtype), rand((13, 7), 10, dtype)
    assert torch.equal(torch.mm(odd_a.to(DEV), odd_b.to(DEV)).cpu(), torch.mm(odd_a, odd_b))
    with pytest.raises(RuntimeError):
        torch.mm(a.to(DEV), a.to(DEV))                   # 200x256 @ 200x256


def test_swiglu_linear_operator():
    dtype = torch.bfloat16
    x, wg, wu = rand((2, 100, 256), 1, dtype), rand((520, 256), 2, dtype, 0.05), rand((520, 256), 3, dtype, 0.05)
    got = paras_nn.swiglu_linear(x.to(DEV), wg.to(DEV), wu.to(DEV))
    assert got.shape == (2, 100, 520)
    close16(got, O.swiglu_linear(x, wg, wu), "swiglu_linear", exact_share=0.97)
    with pytest.raises(RuntimeError):
        paras_nn.swiglu_linear(x.float().to(DEV), wg.float().to(DEV), wu.float().to(DEV))


def test_linearity_at_projection_size():
    # full-size property check (no CPU oracle at this size): A (W1 + W2)^T computed by the kernel
    # equals A W1^T + A W2^T up to the roundings involved, on a 4096-wide projection
    dtype = torch.bfloat16
    g = torch.Generator(device=CUDA).manual_seed(5)
    a = torch.randn(2048, 4096, generator=g, device=CUDA).to(dtype)
    w1 = (torch.randn(4096, 4096, generator=g, device=CUDA) * 0.02).to(dtype)
    w2 = (torch.randn(4096, 4096, generator=g, device=CUDA) * 0.02).to(dtype)
    lhs = abi.gemm(a, (w1.float() + w2.float()).to(dtype)).float()
    rhs = abi.gemm(a, w1).float() + abi.gemm(a, w2).float()
    scale = rhs.abs().mean().item()
    assert (lhs - rhs).abs().max().item() <= 0.05 * scale + 0.1
    assert (lhs - rhs).abs().mean().item() <= 0.01 * scale


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 520, 1000), (1000, 128, 4096), (5, 264, 72),
                                   (16, 6144, 4096), (100, 1032, 520)])   # the last two: the decode-step kernel
def test_rms_norm_folded_into_the_projection(shape, dtype):
    # linear(rms_norm(x, w), W) in one GEMM (row-scale epilogue) against the reference's two steps:
    # paras::rms_norm (fused_ops.cpp:43-88) rounded to 16 bits, then the host GEMM of linear
    # (vision_ops.cpp:248-309).  The fused form rounds W o w instead of the normalised activations,
    # so elements differ by rounding noise of the same size: the bound is 2 ulp of the result plus
    # 2e-2 of the result's scale, and most elements must agree to 1 ulp.
    M, N, K = shape
    x = rand((M, K), 11, dtype, 1.5)
    wn = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(12))).to(dtype)
    w = rand((N, K), 13, dtype, 0.05)
    y, _ = O.rms_norm_fused(x, wn, 1e-6)
    want = O.linear(y, w)
    xd, wnd, wd = x.to(CUDA), wn.to(CUDA), w.to(CUDA)
    # the pieces
    rstd = abi.rms_rstd(xd, 1e-6)
    _, rstd_want = O.rms_norm_fused(x, wn, 1e-6)
    assert torch.allclose(rstd.cpu(), rstd_want, rtol=1e-5, atol=1e-6)
    wf = abi.scale_columns(wd, wnd)
    assert torch.equal(wf.cpu(), (w.float() * wn.float()).to(dtype))
    got = abi.rms_norm_linear(xd, wnd, wd, 1e-6).cpu()
    assert got.shape == want.shape and got.dtype == want.dtype
    g, t = got.double(), want.double()
    scale = t.abs().max().item()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    err = (g - t).abs()
    assert (err <= 2 * ulp * t.abs() + 2e-2 * scale).all(), f"worst {err.max().item():.3e} at scale {scale:.3e}"
    assert (err <= ulp * t.abs() + 1e-3 * scale).double().mean().item() > 0.9
    # the operators on the device give the same bits, folded once or per call
    xp, wnp, wp = x.to(DEV), wn.to(DEV), w.to(DEV)
    o1 = paras_nn.rms_norm_linear(xp, wnp, wp, 1e-6)
    o2 = paras_nn.rms_norm_linear(xp.reshape(1, M, K), None, None, 1e-6, folded_weight=paras_nn.fold_norm_weight(wp, wnp))
    assert torch.equal(o1.cpu(), got) and torch.equal(o2.cpu().reshape(M, N), got)
