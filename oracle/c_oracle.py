"""ctypes face of the plain-C restatement (oracle/paras_oracle.c).

TEST INFRASTRUCTURE ONLY, like everything under oracle/: tests load it to hold the C
restatement to the golden vectors of the unmodified reference and to oracle.py.  ``load()``
builds the shared object with ``make -C oracle cport`` when it is missing or older than its
source.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional, Tuple

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "paras_oracle.c")
LIB = os.path.join(HERE, "_ref", "libparas_oracle_c.so")

_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_lib = None


def build() -> str:
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.check_call(["make", "-C", HERE, "cport"], stdout=subprocess.DEVNULL)
    return LIB


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        i64, dbl, ci, vp = ctypes.c_int64, ctypes.c_double, ctypes.c_int, ctypes.c_void_p
        lib.po_rms_norm_fused.argtypes = [vp, vp, vp, vp, i64, i64, dbl, ci]
        lib.po_rms_norm_fused_backward.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, ci, ci]
        lib.po_rms_norm_composite.argtypes = [vp, vp, vp, i64, i64, dbl, ci]
        lib.po_swiglu_fused.argtypes = [vp, vp, vp, i64, ci]
        lib.po_swiglu_fused_backward.argtypes = [vp, vp, vp, vp, vp, i64, ci]
        lib.po_swiglu_composite.argtypes = [vp, vp, vp, i64, ci]
        lib.po_rotate_half.argtypes = [vp, vp, i64, i64, ci]
        lib.po_rotate_half_backward.argtypes = [vp, vp, i64, i64, ci]
        lib.po_softmax_lastdim.argtypes = [vp, vp, i64, i64, ci]
        lib.po_sdpa.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, dbl, ci, vp, ci, ci]
        for name in ("po_rms_norm_fused", "po_rms_norm_fused_backward", "po_rms_norm_composite",
                     "po_swiglu_fused", "po_swiglu_fused_backward", "po_swiglu_composite",
                     "po_softmax_lastdim"):
            getattr(lib, name).restype = None
        lib.po_f32_to_bf16.argtypes = [ctypes.c_float]
        lib.po_f32_to_bf16.restype = ctypes.c_uint16
        lib.po_f32_to_f16.argtypes = [ctypes.c_float]
        lib.po_f32_to_f16.restype = ctypes.c_uint16
        lib.po_bf16_to_f32.argtypes = [ctypes.c_uint16]
        lib.po_bf16_to_f32.restype = ctypes.c_float
        lib.po_f16_to_f32.argtypes = [ctypes.c_uint16]
        lib.po_f16_to_f32.restype = ctypes.c_float
        _lib = lib
    return _lib


def _code(t: torch.Tensor) -> int:
    if t.dtype not in _CODES:
        raise RuntimeError(f"c oracle: unsupported dtype {t.dtype}")
    return _CODES[t.dtype]


def _c(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous()


def rms_norm_fused(x, weight, eps) -> Tuple[torch.Tensor, torch.Tensor]:
    h = x.size(-1)
    if weight.numel() != h:
        raise RuntimeError("paras rms_norm: weight size must match the last dimension")
    x, weight = _c(x), _c(weight).to(x.dtype)
    rows = x.numel() // h if h else 0
    out = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32)
    load().po_rms_norm_fused(x.data_ptr(), weight.data_ptr(), out.data_ptr(), rstd.data_ptr(),
                             rows, h, float(eps), _code(x))
    return out, rstd


def rms_norm_fused_backward(grad_out, x, weight, rstd):
    h = x.size(-1)
    rows = x.numel() // h if h else 0
    g, x, weight, rstd = _c(grad_out), _c(x), _c(weight), _c(rstd.float())
    gi, gw = torch.empty_like(x), torch.empty_like(weight)
    load().po_rms_norm_fused_backward(g.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                      gi.data_ptr(), gw.data_ptr(), rows, h, _code(x), _code(weight))
    return gi, gw


def rms_norm_composite(x, normalized_shape, weight=None, eps=None):
    n = 1
    for s in normalized_shape:
        n *= int(s)
    nd = len(normalized_shape)
    if nd < 1 or x.dim() < nd or tuple(x.shape[x.dim() - nd:]) != tuple(normalized_shape):
        raise RuntimeError("paras rms_norm: normalized_shape does not match the trailing dims")
    if weight is not None and tuple(weight.shape) != tuple(normalized_shape):
        raise RuntimeError("paras rms_norm: weight shape must equal normalized_shape")
    x = _c(x)
    w = _c(weight).to(x.dtype) if weight is not None else None
    out = torch.empty_like(x)
    load().po_rms_norm_composite(x.data_ptr(), w.data_ptr() if w is not None else None, out.data_ptr(),
                                 x.numel() // n if n else 0, n, 1e-6 if eps is None else float(eps),
                                 _code(x))
    return out


def swiglu_fused(gate, up):
    if gate.shape != up.shape:
        raise RuntimeError("paras swiglu: gate and up must have the same shape")
    gate, up = _c(gate), _c(up)
    out = torch.empty_like(gate)
    load().po_swiglu_fused(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _code(gate))
    return out


def swiglu_fused_backward(grad_out, gate, up):
    dy, gate, up = _c(grad_out), _c(gate), _c(up)
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    load().po_swiglu_fused_backward(dy.data_ptr(), gate.data_ptr(), up.data_ptr(), dg.data_ptr(),
                                    du.data_ptr(), gate.numel(), _code(gate))
    return dg, du


def swiglu_composite(x, gate):
    x, gate = _c(x), _c(gate)
    out = torch.empty_like(x)
    load().po_swiglu_composite(x.data_ptr(), gate.data_ptr(), out.data_ptr(), x.numel(), _code(x))
    return out


def _rotate(fn, x):
    d = x.size(-1)
    x = _c(x)
    out = torch.empty_like(x)
    if fn(x.data_ptr(), out.data_ptr(), x.numel() // d if d else 0, d, _code(x)) != 0:
        raise RuntimeError("paras rotate_half: last dimension must be even")
    return out


def rotate_half(x):
    return _rotate(load().po_rotate_half, x)


def rotate_half_backward(g):
    return _rotate(load().po_rotate_half_backward, g)


def softmax_lastdim(x):
    x = _c(x)
    out = torch.empty_like(x)
    n = x.size(-1)
    load().po_softmax_lastdim(x.data_ptr(), out.data_ptr(), x.numel() // n if n else 0, n, _code(x))
    return out


def sdpa(q, k, v, attn_mask: Optional[torch.Tensor] = None, is_causal: bool = False,
         scale: Optional[float] = None, enable_gqa: bool = False):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("c oracle sdpa: [B, H, L, D] tensors")
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.size(1), k.size(2)
    if Hkv != Hq and not enable_gqa:
        raise RuntimeError("c oracle sdpa: head counts differ without enable_gqa")
    q, k, v = _c(q), _c(k), _c(v)
    kind, mask = 0, None
    if attn_mask is not None:
        full = attn_mask.expand(B, Hq, Lq, Lk)
        if attn_mask.dtype == torch.bool:
            kind, mask = 1, _c(full.to(torch.uint8))
        else:
            kind, mask = 2, _c(full.to(q.dtype))
    out = torch.empty_like(q)
    rc = load().po_sdpa(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, Lq, Lk, D,
                        float(scale) if scale is not None else 1.0 / math.sqrt(float(D)),
                        int(bool(is_causal)), mask.data_ptr() if mask is not None else None, kind,
                        _code(q))
    if rc == 1:
        raise RuntimeError("paras sdpa: arguments the reference rejects")
    if rc:
        raise MemoryError("c oracle sdpa")
    return out
