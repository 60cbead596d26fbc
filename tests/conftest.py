import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "framework-torch-paras_b200", "python"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    # A GPU test on a box without a GPU is an error of the run configuration, not a pass:
    # the hot path has no CPU fallback.  `-m "not gpu"` deselects them here.
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU visible; GPU parity tests run with -m gpu on a B200")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def load_golden(name):
    import torch
    return torch.load(os.path.join(GOLDEN, name + ".pt"))


def golden_names(prefix=""):
    """Fixture names.  Without a prefix: the forward operators' fixtures, the ones the oracle is pinned
    to; the attention-gradient fixtures ("sdpa_grad_...", the reference's autograd output, for which
    the oracle holds no restatement) are listed only when asked for by prefix."""
    names = sorted(f[:-3] for f in os.listdir(GOLDEN) if f.endswith(".pt") and f.startswith(prefix))
    return names if prefix else [n for n in names if not n.startswith("sdpa_grad")]
