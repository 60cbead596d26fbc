"""ctypes bindings of the C ABI in ``include/paras_b200.h`` (``libparas_b200.so``).

This is the same boundary the operator layer (``_C.so``) calls; it is exposed to Python so
that tests, benchmarks and other runtimes can drive the kernels on raw device pointers --
for example on ``torch.cuda`` tensors -- without the ``paras`` device in between.
Every wrapper raises ``RuntimeError`` with the library's message on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

# PARAS_B200_LIB points the bindings at another build of the library (e.g. a tuning variant).
_LIB_PATH = os.environ.get("PARAS_B200_LIB") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "libparas_b200.so")

F32, BF16, F16 = 0, 1, 2
ROUND_ONCE, ROUND_PER_OP = 0, 1
SDPA_REF_SCALE, SDPA_FORCE_SIMT, SDPA_FORCE_TENSOR = 1, 2, 4

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

EXPORTS = [
    "paras_b200_abi_version", "paras_b200_backend_name", "paras_b200_last_error",
    "paras_b200_device_count", "paras_b200_device_name", "paras_b200_device_sm_count",
    "paras_b200_stream", "paras_b200_synchronize", "paras_b200_malloc_async",
    "paras_b200_free_async", "paras_b200_pool_stats", "paras_b200_pool_trim", "paras_b200_pool_set_limit",
    "paras_b200_memcpy_h2d", "paras_b200_memcpy_d2h", "paras_b200_memcpy_d2d",
    "paras_b200_memcpy_peer", "paras_b200_memset", "paras_b200_host_alloc", "paras_b200_host_free",
    "paras_b200_host_is_pinned",
    "paras_b200_strided_copy", "paras_b200_fill", "paras_b200_sdpa_fwd",
    "paras_b200_sdpa_workspace_bytes", "paras_b200_sdpa_mask_is_causal", "paras_b200_sdpa_last_kernel", "paras_b200_rmsnorm_fwd",
    "paras_b200_sdpa_fwd_static_scratch", "paras_b200_sdpa_static_scratch_bytes",
    "paras_b200_rmsnorm_bwd", "paras_b200_swiglu_fwd", "paras_b200_swiglu_bwd",
    "paras_b200_rotate_half", "paras_b200_gemm", "paras_b200_sdpa_fwd_host", "paras_b200_sdpa_bwd",
    "paras_b200_sdpa_split_layout", "paras_b200_selftest_bounded_wait",
    "paras_b200_rms_rstd", "paras_b200_scale_columns", "paras_b200_sdpa_rope_fwd", "paras_b200_rope",
    "paras_b200_sdpa_bwd_general",
]


def pool_set_limit(gpu: int, nbytes: int) -> None:
    """Caps the bytes the pool of CUDA GPU `gpu` may have handed out (0 = no cap)."""
    L = lib()
    L.paras_b200_pool_set_limit.argtypes = [C.c_int, C.c_size_t]
    check(L.paras_b200_pool_set_limit(gpu, nbytes))


class SdpaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("mask", C.c_void_p), ("mask_kind", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Lq", C.c_int32),
        ("Lk", C.c_int32), ("D", C.c_int32),
        ("q_strides", C.c_int64 * 3), ("k_strides", C.c_int64 * 3), ("v_strides", C.c_int64 * 3),
        ("o_strides", C.c_int64 * 3), ("mask_strides", C.c_int64 * 4),
        ("causal", C.c_int32), ("flags", C.c_int32), ("scale", C.c_double),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("gpu", C.c_int32), ("reserved", C.c_int32), ("stream", C.c_void_p),
        ("dropout_p", C.c_double), ("rng_seed", C.c_uint64), ("rng_sequence", C.c_uint64),
        ("dropout_mask", C.c_void_p), ("dropout_mask_strides", C.c_int64 * 4),
        ("dropout_mask_kind", C.c_int32), ("reserved2", C.c_int32), ("attn_out", C.c_void_p),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("b2", C.c_void_p), ("bias", C.c_void_p),
        ("c", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("batch", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
        ("dtype", C.c_int32), ("b_layout", C.c_int32), ("epilogue", C.c_int32), ("gpu", C.c_int32),
        ("stream", C.c_void_p), ("a_layout", C.c_int32), ("reserved", C.c_int32),
        ("row_scale", C.c_void_p),
    ]


class SdpaBwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("dout", C.c_void_p), ("lse", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Lq", C.c_int32),
        ("Lk", C.c_int32), ("D", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32),
        ("scale", C.c_double), ("gpu", C.c_int32), ("reserved", C.c_int32), ("stream", C.c_void_p),
    ]


GEMM_B_NK, GEMM_B_KN = 0, 1
GEMM_EPI_NONE, GEMM_EPI_BIAS, GEMM_EPI_SWIGLU, GEMM_EPI_ROWSCALE = 0, 1, 2, 5

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: build it with framework-torch-paras_b200/build.py")
        L = C.CDLL(_LIB_PATH)
        L.paras_b200_last_error.restype = C.c_char_p
        L.paras_b200_backend_name.restype = C.c_char_p
        L.paras_b200_sdpa_last_kernel.restype = C.c_char_p
        L.paras_b200_sdpa_fwd.argtypes = [C.POINTER(SdpaArgs)]
        L.paras_b200_sdpa_workspace_bytes.argtypes = [C.POINTER(SdpaArgs), C.POINTER(C.c_size_t)]
        L.paras_b200_sdpa_fwd_static_scratch.argtypes = [C.POINTER(SdpaArgs)]
        L.paras_b200_gemm.argtypes = [C.POINTER(GemmArgs)]
        L.paras_b200_sdpa_fwd_host.argtypes = [C.POINTER(SdpaArgs)]
        L.paras_b200_sdpa_bwd.argtypes = [C.POINTER(SdpaBwdArgs)]
        L.paras_b200_rmsnorm_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_int64, C.c_int64, C.c_double, C.c_int, C.c_int, C.c_void_p]
        L.paras_b200_rmsnorm_bwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
        L.paras_b200_swiglu_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                            C.c_int, C.c_int, C.c_void_p]
        L.paras_b200_swiglu_bwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        L.paras_b200_rotate_half.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                             C.c_int, C.c_int, C.c_void_p]
        L.paras_b200_memcpy_h2d.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]
        L.paras_b200_memcpy_d2h.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.paras_b200_malloc_async.argtypes = [C.c_int, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p)]
        L.paras_b200_free_async.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
        L.paras_b200_synchronize.argtypes = [C.c_int]
        L.paras_b200_stream.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        L.paras_b200_host_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
        L.paras_b200_host_free.argtypes = [C.c_void_p]
        L.paras_b200_host_is_pinned.argtypes = [C.c_void_p]
        L.paras_b200_sdpa_split_layout.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_size_t),
                                                   C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.paras_b200_selftest_bounded_wait.argtypes = [C.c_int, C.c_uint32, C.POINTER(C.c_int)]
        L.paras_b200_sdpa_rope_fwd.argtypes = [C.POINTER(SdpaArgs), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        L.paras_b200_rope.argtypes = [C.c_int, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_void_p]
        L.paras_b200_rms_rstd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_double,
                                          C.c_int, C.c_void_p]
        L.paras_b200_scale_columns.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                               C.c_int, C.c_void_p]
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(lib().paras_b200_last_error().decode())


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError(f"paras: unsupported dtype {t.dtype}") from None


_LEGACY_DEFAULT_STREAM = 1  # cudaStreamLegacy: a NULL stream argument means "the library's own"


def _stream_of(t: torch.Tensor, stream) -> int:
    """The stream the launch goes to: torch's current stream of the tensor's device, so that
    the kernel is ordered with the torch work that produced its inputs and reads its outputs."""
    if stream is not None:
        return int(stream)
    if t.is_cuda:
        return int(torch.cuda.current_stream(t.device).cuda_stream) or _LEGACY_DEFAULT_STREAM
    return 0


def _gpu_of(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("paras abi: expected a CUDA tensor (raw device memory)")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def sdpa_args(q, k, v, out, *, causal=False, scale=None, mask=None, lse=None, flags=0,
              workspace=None, stream=None) -> SdpaArgs:
    """Fills a ``paras_sdpa_args`` from [B,H,L,D] tensors (any B/H/L strides, unit D stride)."""
    for t in (q, k, v, out):
        if t.dim() != 4 or (t.size(-1) > 1 and t.stride(-1) != 1):
            raise RuntimeError("paras abi: expected [B,H,L,D] tensors with a contiguous last dim")
    a = SdpaArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.dtype = dtype_code(q)
    a.B, a.Hq, a.Lq, a.D = q.shape
    a.Hkv, a.Lk = k.shape[1], k.shape[2]
    for i in range(3):
        a.q_strides[i], a.k_strides[i] = q.stride(i), k.stride(i)
        a.v_strides[i], a.o_strides[i] = v.stride(i), out.stride(i)
    if mask is not None:
        m = mask
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m = m.expand(q.shape[0], q.shape[1], q.shape[2], k.shape[2])
        a.mask = m.data_ptr()
        a.mask_kind = 1 if m.dtype == torch.bool else (2 if m.dtype == q.dtype else 3)
        if a.mask_kind == 3 and m.dtype != torch.float32:
            raise RuntimeError("paras abi: additive mask must have the tensors' dtype or float32")
        for i in range(4):
            a.mask_strides[i] = m.stride(i)
        a._keep = m
    a.causal = 1 if causal else 0
    a.flags = flags
    a.scale = float(scale) if scale is not None else 1.0 / (q.shape[-1] ** 0.5)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    a.gpu = _gpu_of(q)
    a.stream = _stream_of(q, stream)
    return a


def sdpa_fwd(q, k, v, *, causal=False, scale=None, mask=None, return_lse=False, flags=0,
             out=None, workspace=None, stream=None, dropout_p=0.0, rng=None, dropout_mask=None,
             return_weights=False):
    """softmax(q k^T * scale [+mask]) v through ``paras_b200_sdpa_fwd``.  ``dropout_p`` with
    ``rng=(seed, sequence)`` draws the reference's Philox stream, ``dropout_mask`` multiplies a given
    mask in instead, ``return_weights`` also returns the [B,Hq,Lq,Lk] attention weights."""
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if return_lse else None
    a = sdpa_args(q, k, v, out, causal=causal, scale=scale, mask=mask, lse=lse, flags=flags,
                  workspace=workspace, stream=stream)
    weights = None
    a.dropout_p = float(dropout_p)
    if rng is not None:
        a.rng_seed, a.rng_sequence = int(rng[0]), int(rng[1])
    if dropout_mask is not None:
        m = dropout_mask
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m = m.expand(q.shape[0], q.shape[1], q.shape[2], k.shape[2])
        a.dropout_mask = m.data_ptr()
        a.dropout_mask_kind = 1 if m.dtype == torch.bool else (2 if m.dtype == q.dtype else 3)
        for i in range(4):
            a.dropout_mask_strides[i] = m.stride(i)
        a._keep_dm = m
    if return_weights:
        weights = torch.empty((q.shape[0], q.shape[1], q.shape[2], k.shape[2]), dtype=q.dtype, device=q.device)
        a.attn_out = weights.data_ptr()
    check(lib().paras_b200_sdpa_fwd(C.byref(a)))
    res = (out,) + ((lse,) if return_lse else ()) + ((weights,) if return_weights else ())
    return res if len(res) > 1 else out


def sdpa_bwd_general(dout, q, k, v, *, causal=False, scale=None, mask=None, flags=0, stream=None,
                     dropout_p=0.0, rng=None, dropout_mask=None):
    """(dq, dk, dv) through ``paras_b200_sdpa_bwd_general``: the gradient of ``sdpa_fwd`` called with the
    same arguments (mask, dropout with the same ``rng`` or ``dropout_mask``), any dtype, any head dim."""
    if dout.dim() != 4 or (dout.size(-1) > 1 and dout.stride(-1) != 1):
        raise RuntimeError("paras abi: dout must be [B,H,L,D] with a contiguous last dim")
    dq, dk, dv = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype, device=k.device), \
        torch.empty(v.shape, dtype=v.dtype, device=v.device)
    a = sdpa_args(q, k, v, dq, causal=causal, scale=scale, mask=mask, flags=flags, stream=stream)
    a.dropout_p = float(dropout_p)
    if rng is not None:
        a.rng_seed, a.rng_sequence = int(rng[0]), int(rng[1])
    if dropout_mask is not None:
        m = dropout_mask
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m = m.expand(q.shape[0], q.shape[1], q.shape[2], k.shape[2])
        a.dropout_mask = m.data_ptr()
        a.dropout_mask_kind = 1 if m.dtype == torch.bool else (2 if m.dtype == q.dtype else 3)
        for i in range(4):
            a.dropout_mask_strides[i] = m.stride(i)
        a._keep_dm = m
    st = (C.c_int64 * 3)(dout.stride(0), dout.stride(1), dout.stride(2))
    L = lib()
    L.paras_b200_sdpa_bwd_general.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    check(L.paras_b200_sdpa_bwd_general(C.byref(a), dout.data_ptr(), st, dq.data_ptr(), dk.data_ptr(), dv.data_ptr()))
    return dq, dk, dv


def sdpa_rope_fwd(q, k, v, cos, sin, *, causal=False, scale=None, q_pos0=0, flags=0, out=None, stream=None):
    """sdpa(rope(q), rope(k), v) through ``paras_b200_sdpa_rope_fwd``; cos / sin [rows, D] in q's dtype."""
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    assert cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape and cos.dtype == q.dtype
    a = sdpa_args(q, k, v, out, causal=causal, scale=scale, flags=flags, stream=stream)
    check(lib().paras_b200_sdpa_rope_fwd(C.byref(a), cos.data_ptr(), sin.data_ptr(), cos.shape[0], q_pos0))
    return out


def rope(x, cos, sin, *, pos0=0, stream=None):
    """x * cos + rotate_half(x) * sin for x [B, H, L, D] (any B/H/L strides), rounding per operation."""
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    st = (C.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
    check(lib().paras_b200_rope(_gpu_of(x), x.data_ptr(), st, cos.data_ptr(), sin.data_ptr(), out.data_ptr(),
                                x.shape[0], x.shape[1], x.shape[2], x.shape[3], pos0, dtype_code(x),
                                _stream_of(x, stream)))
    return out


def sdpa_fwd_host(q, k, v, *, causal=False, scale=None, flags=0, out=None, gpu=0):
    """Attention on host tensors through ``paras_b200_sdpa_fwd_host``: batch chunks are copied
    in, computed and copied out as a pipeline on GPU ``gpu``.  Pass page-locked tensors
    (``pin_memory()``) for full overlap; ``out`` (host, same shape as q) is created pinned when
    omitted."""
    for t in (q, k, v):
        if t.device.type != "cpu" or not t.is_contiguous():
            raise RuntimeError("paras abi: sdpa_fwd_host takes contiguous host tensors")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    a = SdpaArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.dtype = dtype_code(q)
    a.B, a.Hq, a.Lq, a.D = q.shape
    a.Hkv, a.Lk = k.shape[1], k.shape[2]
    for i in range(3):
        a.q_strides[i], a.k_strides[i] = q.stride(i), k.stride(i)
        a.v_strides[i], a.o_strides[i] = v.stride(i), out.stride(i)
    a.causal = 1 if causal else 0
    a.flags = flags
    a.scale = float(scale) if scale is not None else 1.0 / (q.shape[-1] ** 0.5)
    a.gpu = gpu
    a.stream = None
    check(lib().paras_b200_sdpa_fwd_host(C.byref(a)))
    return out


SDPA_BWD_COMPOSITE = 1


def sdpa_bwd(dout, q, k, v, out, lse, *, causal=False, scale=None, stream=None, composite=False):
    """(dq, dk, dv) through ``paras_b200_sdpa_bwd``; contiguous [B,H,L,D] tensors, ``lse`` from
    ``sdpa_fwd(..., return_lse=True)`` with the same causal flag and scale.  ``composite`` forces
    the five-GEMM path that other head dims than 128 / 64 take."""
    for t in (dout, q, k, v, out):
        if not t.is_contiguous():
            raise RuntimeError("paras abi: sdpa_bwd takes contiguous tensors")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    a = SdpaBwdArgs()
    a.q, a.k, a.v, a.out, a.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr()
    a.lse = lse.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.B, a.Hq, a.Lq, a.D = q.shape
    a.Hkv, a.Lk = k.shape[1], k.shape[2]
    a.dtype = dtype_code(q)
    a.causal = 1 if causal else 0
    a.scale = float(scale) if scale is not None else 1.0 / (q.shape[-1] ** 0.5)
    a.gpu = _gpu_of(q)
    a.reserved = SDPA_BWD_COMPOSITE if composite else 0
    a.stream = _stream_of(q, stream)
    check(lib().paras_b200_sdpa_bwd(C.byref(a)))
    return dq, dk, dv


def sdpa_fwd_static_scratch(q, k, v, *, causal=False, scale=None, mask=None, flags=0, out=None,
                            stream=None):
    """Attention through ``paras_b200_sdpa_fwd_static_scratch``: for callers that must not
    allocate device memory while they run (the split-KV scratch is a fixed array inside the
    library).  ``out`` should be passed in by such a caller; it is only created here when
    omitted."""
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    a = sdpa_args(q, k, v, out, causal=causal, scale=scale, mask=mask, flags=flags, stream=stream)
    check(lib().paras_b200_sdpa_fwd_static_scratch(C.byref(a)))
    return out


def rms_rstd(x, eps=1e-6, *, stream=None):
    """1 / sqrt(mean(x^2, -1) + eps) per row of a contiguous [rows, H] tensor, fp32."""
    h = x.shape[-1]
    rows = x.numel() // h if h else 0
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(lib().paras_b200_rms_rstd(_gpu_of(x), x.data_ptr(), rstd.data_ptr(), rows, h, float(eps), dtype_code(x),
                                    _stream_of(x, stream)))
    return rstd


def scale_columns(weight, scale, *, stream=None):
    """weight[n, k] * scale[k] with one rounding (the RMSNorm weight folded into a projection weight)."""
    assert weight.is_contiguous() and scale.is_contiguous() and weight.shape[-1] == scale.numel()
    out = torch.empty_like(weight)
    check(lib().paras_b200_scale_columns(_gpu_of(weight), weight.data_ptr(), scale.data_ptr(), out.data_ptr(),
                                         weight.numel() // scale.numel(), scale.numel(), dtype_code(weight),
                                         _stream_of(weight, stream)))
    return out


def rms_norm_linear(x, norm_weight, weight, eps=1e-6, *, folded_weight=None, stream=None):
    """linear(rms_norm(x, norm_weight), weight) without writing the normalised activations: rstd in one
    read of x, the norm weight folded into the projection weight (pass ``folded_weight`` to reuse it),
    and the GEMM's epilogue scaling its rows by rstd."""
    wf = folded_weight if folded_weight is not None else scale_columns(weight, norm_weight, stream=stream)
    x2 = x.reshape(-1, x.shape[-1])
    out = gemm(x2, wf, row_scale=rms_rstd(x2, eps, stream=stream), stream=stream)
    return out.reshape(*x.shape[:-1], wf.shape[0])


def gemm(a, b, *, b_layout=GEMM_B_NK, a_transposed=False, bias=None, up_weight=None, row_scale=None, out=None,
         stream=None):
    """``paras_b200_gemm`` on 2-D ([M,K]) or 3-D ([batch,M,K]) operands with contiguous rows.

    ``b_layout=GEMM_B_NK``: b is [N,K] (a Linear weight), result a @ b^T;
    ``GEMM_B_KN``: b is [K,N], result a @ b.  ``bias`` [N] adds a bias; ``up_weight`` [N,K]
    makes b the gate weight of a fused SwiGLU: swiglu(a @ b^T, a @ up_weight^T).
    """
    batched = a.dim() == 3
    a3 = a if batched else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    if a3.stride(-1) != 1 or b3.stride(-1) != 1:
        raise RuntimeError("paras abi: gemm operands need contiguous rows")
    if a_transposed:  # a is [.., K, M]: the product is a^T @ b
        Bt, K, M = a3.shape
    else:
        Bt, M, K = a3.shape
    N = b3.shape[1] if b_layout == GEMM_B_NK else b3.shape[2]
    if out is None:
        out = torch.empty((Bt, M, N) if batched else (M, N), dtype=a.dtype, device=a.device)
    c3 = out if out.dim() == 3 else out.unsqueeze(0)
    g = GemmArgs()
    g.a, g.b, g.c = a3.data_ptr(), b3.data_ptr(), c3.data_ptr()
    g.b2 = up_weight.data_ptr() if up_weight is not None else None
    g.bias = bias.data_ptr() if bias is not None else None
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb, g.ldc = a3.stride(1), b3.stride(1), c3.stride(1)
    g.batch = Bt
    g.stride_a, g.stride_c = a3.stride(0), c3.stride(0)
    g.stride_b = b3.stride(0) if b3.shape[0] > 1 else 0
    g.dtype = dtype_code(a)
    g.b_layout = b_layout
    g.a_layout = 1 if a_transposed else 0
    g.epilogue = GEMM_EPI_SWIGLU if up_weight is not None else (GEMM_EPI_BIAS if bias is not None else GEMM_EPI_NONE)
    if row_scale is not None:
        if g.epilogue != GEMM_EPI_NONE:
            raise RuntimeError("paras abi: row_scale cannot be combined with another epilogue")
        g.epilogue = GEMM_EPI_ROWSCALE
        g.row_scale = row_scale.data_ptr()
    g.gpu = _gpu_of(a)
    g.stream = _stream_of(a, stream)
    check(lib().paras_b200_gemm(C.byref(g)))
    return out


def sdpa_workspace_bytes(q, k, v, *, causal=False, flags=0) -> int:
    a = sdpa_args(q, k, v, q, causal=causal, flags=flags)
    n = C.c_size_t(0)
    check(lib().paras_b200_sdpa_workspace_bytes(C.byref(a), C.byref(n)))
    return int(n.value)


def sdpa_mask_is_causal(mask, dtype, scale=None, head_dim=128) -> bool:
    """Whether a 2-D [Lq, Lk] mask (bool, `dtype`, or fp32) is the causal mask written out; waits for the GPU."""
    assert mask.dim() == 2 and mask.stride(1) == 1
    kind = 1 if mask.dtype == torch.bool else (2 if mask.dtype == dtype else 3)
    res = C.c_int(0)
    check(lib().paras_b200_sdpa_mask_is_causal(_gpu_of(mask), C.c_void_p(mask.data_ptr()), kind, _DT[dtype],
                                               C.c_int64(mask.stride(0)), mask.shape[0], mask.shape[1],
                                               C.c_double(scale if scale is not None else head_dim ** -0.5),
                                               C.c_void_p(_stream_of(mask, None)), C.byref(res)))
    return bool(res.value)


def sdpa_split_layout(rows: int, D: int, splits: int):
    """(ml_offset, o_offset, bytes) of the split-KV scratch; host arithmetic, needs no GPU."""
    ml, o, n = C.c_size_t(0), C.c_size_t(0), C.c_size_t(0)
    check(lib().paras_b200_sdpa_split_layout(rows, D, splits, C.byref(ml), C.byref(o), C.byref(n)))
    return int(ml.value), int(o.value), int(n.value)


def selftest_bounded_wait(gpu: int, limit_us: int = 1000):
    """Runs the bounded-wait self-test kernel; returns (status code, raw status word)."""
    word = C.c_int(0)
    st = lib().paras_b200_selftest_bounded_wait(gpu, limit_us, C.byref(word))
    return int(st), int(word.value)


def sdpa_last_kernel() -> str:
    return lib().paras_b200_sdpa_last_kernel().decode()


def rmsnorm_fwd(x, weight, eps=1e-6, *, mode=ROUND_ONCE, return_rstd=False, out=None, stream=None):
    h = x.shape[-1]
    rows = x.numel() // h if h else 0
    assert x.is_contiguous() and (weight is None or weight.is_contiguous())
    if out is None:
        out = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if return_rstd else None
    check(lib().paras_b200_rmsnorm_fwd(
        _gpu_of(x), x.data_ptr(), weight.data_ptr() if weight is not None else None, out.data_ptr(),
        rstd.data_ptr() if rstd is not None and rows else None, rows, h, float(eps), dtype_code(x),
        mode, _stream_of(x, stream)))
    return (out, rstd) if return_rstd else out


def rmsnorm_bwd(grad_out, x, weight, rstd, *, stream=None):
    h = x.shape[-1]
    rows = x.numel() // h if h else 0
    gx = torch.empty_like(x)
    gw = torch.empty_like(weight)
    check(lib().paras_b200_rmsnorm_bwd(
        _gpu_of(x), grad_out.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
        gx.data_ptr(), gw.data_ptr(), rows, h, dtype_code(x), _stream_of(x, stream)))
    return gx, gw


def swiglu_fwd(gate, up, *, mode=ROUND_ONCE, out=None, stream=None):
    assert gate.is_contiguous() and up.is_contiguous() and gate.shape == up.shape
    if out is None:
        out = torch.empty_like(gate)
    check(lib().paras_b200_swiglu_fwd(_gpu_of(gate), gate.data_ptr(), up.data_ptr(), out.data_ptr(),
                                      gate.numel(), dtype_code(gate), mode, _stream_of(gate, stream)))
    return out


def swiglu_bwd(grad_out, gate, up, *, stream=None):
    gg, gu = torch.empty_like(gate), torch.empty_like(up)
    check(lib().paras_b200_swiglu_bwd(_gpu_of(gate), grad_out.data_ptr(), gate.data_ptr(), up.data_ptr(),
                                      gg.data_ptr(), gu.data_ptr(), gate.numel(), dtype_code(gate),
                                      _stream_of(gate, stream)))
    return gg, gu


def rotate_half(x, *, backward=False, stream=None):
    assert x.is_contiguous()
    d = x.shape[-1]
    out = torch.empty_like(x)
    check(lib().paras_b200_rotate_half(_gpu_of(x), x.data_ptr(), out.data_ptr(), x.numel() // d if d else 0,
                                       d, dtype_code(x), 1 if backward else 0, _stream_of(x, stream)))
    return out
