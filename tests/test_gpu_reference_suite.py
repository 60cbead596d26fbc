"""The reference's OWN test files for the hot path, run as they are against this library's
`paras:1` device (the first B200): tests/test_attention_norm_ops.py and tests/test_fused_ops.py
of the reference, driven by its tests/run_all.py and tests/common.py (run_all.py:26-75 runs
every `test_*` function of a module with `torch.manual_seed(0)` and returns the number of
failures as its exit code; common.py:12 takes the device from TORCH_PARAS_DEVICE).

Nothing of the reference is committed here.  The four files are read from a checkout of the
reference (PARAS_REFERENCE_DIR, or a folder `reference` beside this repository), else from
oracle/_ref/tests/ where `make -C oracle reftests` put unchanged copies; they are copied to
a temporary folder (so that run_all.py's own `../python` path entry finds nothing and the
`torch_paras` of THIS repository is the one imported) and run in a child process.  The only
thing set from outside is run_all.MODULES: the reference's other six modules test its generic
operator library, which is not part of the hot path.
"""
import os
import shutil
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

FILES = ["common.py", "run_all.py", "test_attention_norm_ops.py", "test_fused_ops.py"]
MODULES = ["test_fused_ops", "test_attention_norm_ops"]


def _reference_tests_dir():
    cands = []
    if os.environ.get("PARAS_REFERENCE_DIR"):
        cands.append(os.path.join(os.environ["PARAS_REFERENCE_DIR"], "tests"))
    cands.append(os.path.join(os.path.dirname(ROOT), "reference", "tests"))
    cands.append(os.path.join(ROOT, "oracle", "_ref", "tests"))
    for d in cands:
        if all(os.path.exists(os.path.join(d, f)) for f in FILES):
            return d
    return None


def test_reference_hot_path_tests_pass_unchanged_on_the_b200_device(tmp_path):
    src = _reference_tests_dir()
    if src is None:
        pytest.skip("the reference's test files are not here: neither a checkout of the reference "
                    "nor oracle/_ref/tests (make -C oracle reftests REF=...)")
    work = tmp_path / "tests"
    work.mkdir()
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), work / f)
    driver = ("import sys; sys.path.insert(0, %r); import run_all; run_all.MODULES = %r; "
              "sys.exit(run_all.main())" % (str(work), MODULES))
    env = dict(os.environ)
    env["TORCH_PARAS_DEVICE"] = "paras:1"
    env["PYTHONPATH"] = os.path.join(ROOT, "framework-torch-paras_b200", "python") + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", driver], cwd=str(work), env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=600)
    print(r.stdout[-6000:])
    assert "paras-b200" in r.stdout, "the run did not go through this repository's torch_paras"
    assert "FAIL" not in r.stdout and r.returncode == 0, f"run_all exit code {r.returncode}"
    # 6 tests in test_fused_ops + 18 in test_attention_norm_ops
    assert "RESULTS: 24 passed, 0 failed" in r.stdout
