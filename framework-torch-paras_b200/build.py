"""Builds the two native pieces of the package, in-tree:

  python/torch_paras/libparas_b200.so   hand-written CUDA kernels + C ABI (nvcc, sm_100a only)
  python/torch_paras/_C.so              the `paras` PrivateUse1 device + operator registrations
                                        (g++ against the installed torch), linked to the above

    python framework-torch-paras_b200/build.py [--force] [--verbose] [--only lib|ext]

nvcc cross-compiles for sm_100a without a GPU.  Objects go to build/ (git-ignored); a
target is rebuilt when any of its sources or headers is newer than it.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
INCLUDE = os.path.join(ROOT, "include")
CSRC = os.path.join(HERE, "csrc")
PKG = os.path.join(HERE, "python", "torch_paras")
OBJ = os.path.join(HERE, "build")

CUDA_SOURCES = ["runtime.cu", "elementwise.cu", "rmsnorm.cu", "sdpa.cu", "sdpa_simt.cu",
                "sdpa_tc.cu", "sdpa_decode.cu", "gemm_tc.cu", "gemm_tc2.cu", "gemm_skinny.cu", "sdpa_bwd.cu", "sdpa_bwd_tc.cu", "sdpa_bwd_general.cu", "sdpa_weights.cu", "selftest.cu"]
EXT_SOURCES = ["core/device_runtime.cpp", "ops/lifecycle_ops.cpp", "ops/attention_ops.cpp",
               "ops/norm_glu_ops.cpp", "ops/matmul_ops.cpp", "python/module.cpp"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-diag-suppress", "177,550"]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers(*dirs: str) -> list[str]:
    out = []
    for d in dirs:
        for base, _, files in os.walk(d):
            out += [os.path.join(base, f) for f in files if f.endswith((".h", ".cuh", ".hpp"))]
    return out


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout}")
    if verbose and r.stdout.strip():
        print(r.stdout)


def nvcc_path() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def build_lib(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers(os.path.join(CSRC, "compat"), INCLUDE)
    out = os.path.join(PKG, "libparas_b200.so")
    jobs, objs = [], []
    for src in CUDA_SOURCES:
        s = os.path.join(CSRC, "compat", src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([nvcc_path(), *NVCC_FLAGS, "-I", INCLUDE, "-I", os.path.join(CSRC, "compat"),
                         "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(out, objs):
        # the C ABI is exported through a version script; everything else stays hidden
        vs = os.path.join(OBJ, "exports.map")
        with open(vs, "w") as f:
            f.write("{ global: paras_b200_*; local: *; };\n")
        _run([nvcc_path(), "-shared", "-o", out, *objs, "-Xlinker", f"--version-script={vs}"],
             verbose)
    return out


def build_ext(force: bool = False, verbose: bool = False) -> str:
    import pybind11
    import torch

    os.makedirs(OBJ, exist_ok=True)
    tdir = os.path.dirname(torch.__file__)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    hdrs = _headers(os.path.join(CSRC, "core"), INCLUDE)
    out = os.path.join(PKG, "_C.so")
    flags = ["-std=c++17", "-O2", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             "-DTORCH_API_INCLUDE_EXTENSION_H", "-DTORCH_EXTENSION_NAME=_C",
             "-I", CSRC, "-I", INCLUDE,
             "-isystem", os.path.join(tdir, "include"),
             "-isystem", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
             "-isystem", sysconfig.get_paths()["include"], "-isystem", pybind11.get_include()]
    jobs, objs = [], []
    for src in EXT_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, "ext_" + src.replace("/", "_").replace(".cpp", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append(["g++", *flags, "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = os.path.join(PKG, "libparas_b200.so")
    if force or jobs or _newer(out, objs + [lib]):
        _run(["g++", "-shared", "-o", out, *objs, "-L", PKG, "-lparas_b200",
              "-L", os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10",
              "-lpthread", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{os.path.join(tdir, 'lib')}"], verbose)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_lib(force, verbose)
    build_ext(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--only", choices=["lib", "ext"])
    a = ap.parse_args()
    if a.only in (None, "lib"):
        print("built", build_lib(a.force, a.verbose))
    if a.only in (None, "ext"):
        print("built", build_ext(a.force, a.verbose))
