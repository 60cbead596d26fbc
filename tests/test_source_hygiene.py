"""Rules the sources keep, checked as text (no GPU): calls this code base does not make, and comments that
stand on their own."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SKIP_DIRS = {".git", "_work", "gpurun_out", "build", "__pycache__", ".pytest_cache", "_ref", ".hypothesis"}
EXTS = (".cu", ".cuh", ".cpp", ".h", ".c", ".py")


def sources():
    for base, dirs, files in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in SKIP_DIRS]
        for f in files:
            if f.endswith(EXTS) or f == "Makefile":
                path = os.path.join(base, f)
                if os.path.abspath(path) != os.path.abspath(__file__):
                    yield path


def test_no_batched_memcpy_calls_and_no_multicast_loads():
    # the names are assembled here so that this file does not contain them either
    batched = ["cu" + "daMemcpy" + tail for tail in ("BatchAsync", "3DBatchAsync")] + \
              ["cu" + "Memcpy" + tail for tail in ("BatchAsync", "3DBatchAsync")]
    multicast = ".multi" + "cast::cluster"
    for path in sources():
        text = open(path, errors="replace").read()
        for name in batched:
            assert name not in text, f"{path} names {name}"
        for n, line in enumerate(text.splitlines(), 1):
            if multicast in line and "cp.async" in line:
                raise AssertionError(f"{path}:{n}: a bulk or TMA load with cluster multicast")


def test_comments_do_not_point_outside_the_sources():
    words = [w + ".md" for w in ("DESIGN", "SURVEY", "VERDICT", "ADVICE", "BASELINE")] + ["gpu" + "run", "/ro" + "ot/"]
    pat = re.compile("|".join(re.escape(w) for w in words))
    for path in sources():
        for n, line in enumerate(open(path, errors="replace").read().splitlines(), 1):
            assert not pat.search(line), f"{path}:{n}: {line.strip()[:120]}"
