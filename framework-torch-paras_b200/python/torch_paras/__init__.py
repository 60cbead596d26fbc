"""B200-native hot path behind the ``paras`` PyTorch device.

Importing this package registers the ``paras`` device (PyTorch's PrivateUse1 backend,
renamed) exactly as the reference package does (python/torch_paras/__init__.py:117-136):

    import torch, torch_paras
    q = q_cpu.to("paras:1")                     # device 1.. = the B200 GPUs, device 0 = host
    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)

``F.scaled_dot_product_attention``, ``F.rms_norm`` / ``torch.ops.aten.rms_norm``,
``torch.ops.paras.{rms_norm,swiglu,rotate_half}`` and ``torch.ops.torch_paras.swiglu`` on
``paras:1..N`` run hand-written sm_100a CUDA kernels from ``libparas_b200.so``.  There is no
CPU fallback for these operators: without the compiled extension the import fails, and
without a GPU the operators raise.
"""
import os
import types

import torch

_here = os.path.dirname(os.path.abspath(__file__))
if not os.path.exists(os.path.join(_here, "libparas_b200.so")):
    raise ImportError(
        "torch_paras: libparas_b200.so is missing next to the package; build it with "
        "`python framework-torch-paras_b200/build.py` (needs nvcc for sm_100a)")

from . import _C  # noqa: E402
from . import nn  # noqa: E402,F401

__all__ = [
    "device_count", "gpu_count", "is_available", "synchronize", "manual_seed", "manual_seed_all",
    "empty_cache", "device_name", "backend_name", "is_gpu_device", "memory_allocated",
    "memory_cached", "get_amp_supported_dtype", "nn",
]


def device_count() -> int:
    """How many ``paras`` devices there are: index 0 is the host, 1.. are the visible GPUs."""
    return _C.device_count()


def gpu_count() -> int:
    return _C.gpu_count()


def is_available() -> bool:
    return device_count() > 0


def backend_name() -> str:
    return _C.backend_name()


def device_name(device: int = 0) -> str:
    return _C.device_name(device)


def is_gpu_device(device: int) -> bool:
    return _C.is_gpu_device(device)


def synchronize(device: int | None = None) -> None:
    """Waits for everything launched so far on ``device`` -- on every device when none is given.  This
    is also where a kernel's bounded wait that ran out is reported (RuntimeError)."""
    if device is None:
        _C.synchronize_all()
    else:
        _C.synchronize(device)


def manual_seed(seed: int, device: int | None = None) -> None:
    if device is None:
        _C.manual_seed_all(seed)
    else:
        _C.manual_seed(device, seed)


def manual_seed_all(seed: int) -> None:
    _C.manual_seed_all(seed)


def empty_cache() -> None:
    """Gives the memory the per-GPU stream-ordered pools hold but do not use back to the driver
    (``PTSYCL_NO_CACHE=1`` in the environment keeps the pools from caching in the first place)."""
    _C.empty_cache()


def memory_allocated(device: int = 0) -> int:
    return _C.allocated_bytes(device)


def memory_cached(device: int = 0) -> int:
    return _C.cached_bytes(device)


def set_memory_limit(nbytes: int, device: int = 1) -> None:
    """Caps the device memory `paras:device` (1..N) may hold at any time; 0 lifts the cap.  An
    allocation that would pass it raises RuntimeError("... out of memory ...") like a full device."""
    if device < 1:
        raise ValueError("paras:0 is the host; memory limits apply to paras:1..N")
    from . import abi
    abi.pool_set_limit(device - 1, int(nbytes))


def get_amp_supported_dtype() -> list[torch.dtype]:
    return [torch.float16, torch.bfloat16, torch.float32]


def _register() -> None:
    torch.utils.rename_privateuse1_backend("paras")
    mod = types.ModuleType("torch.paras")
    mod.device_count = device_count
    mod.is_available = is_available
    mod.synchronize = synchronize
    mod.manual_seed = manual_seed
    mod.manual_seed_all = manual_seed_all
    mod.empty_cache = empty_cache
    mod.device_name = device_name
    mod.is_bad_fork = _C.is_bad_fork
    mod._is_in_bad_fork = _C.is_bad_fork
    mod.get_amp_supported_dtype = get_amp_supported_dtype
    torch._register_device_module("paras", mod)
    torch.utils.generate_methods_for_privateuse1_backend(
        for_tensor=True, for_module=True, for_storage=False)


_register()
