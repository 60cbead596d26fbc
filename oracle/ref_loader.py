"""Loads the UNMODIFIED reference build (oracle/_ref/_C.so, made by oracle/Makefile)
and brings up its ``paras`` PrivateUse1 device, without the reference's Python package.

Test infrastructure only.  The reference library and the product library both define
the ``paras`` operator namespace and both rename PrivateUse1, so they can never share a
process: everything that needs the real reference runs this module in a child process
(see ``oracle/ref_run.py``).

What the reference's own package does at import (python/torch_paras/__init__.py:117-136)
is restated here in the few lines that matter for the hot path: load the extension,
rename the backend, register a device module, generate ``tensor.paras()``.
"""
import importlib.machinery
import importlib.util
import os
import types

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(_HERE, "_ref", "_C.so")


def available() -> bool:
    return os.path.exists(REF_SO)


def load():
    """Returns the reference's pybind module ``_C`` with device ``paras:0`` usable."""
    if not available():
        raise RuntimeError(
            "reference build missing: run `make -C oracle ref` where the reference "
            "sources are present")
    loader = importlib.machinery.ExtensionFileLoader("_C", REF_SO)
    spec = importlib.util.spec_from_loader("_C", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)

    torch.utils.rename_privateuse1_backend("paras")
    dm = types.ModuleType("torch.paras")
    dm.device_count = mod.device_count
    dm.is_available = lambda: mod.device_count() > 0
    dm.synchronize = lambda device=None: (
        mod.synchronize_all() if device is None else mod.synchronize(device))
    dm.is_bad_fork = mod.is_bad_fork
    dm._is_in_bad_fork = mod.is_bad_fork
    dm.manual_seed_all = mod.manual_seed_all
    dm.get_amp_supported_dtype = lambda: [torch.float16, torch.float32]
    torch._register_device_module("paras", dm)
    torch.utils.generate_methods_for_privateuse1_backend(
        for_tensor=True, for_module=True, for_storage=False)
    return mod
