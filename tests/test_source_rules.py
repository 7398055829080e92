"""Rules the product sources must keep, checked on the text (no GPU, no build).

* The shipped library reads no environment variable: every getenv in the kernels' sources sits inside an
  `#ifdef ULLM_CUDA_TUNING` block (a stray variable must not change a drop-in backend's answers).
* No TMA or bulk load is issued with cluster multicast, and none of the batched-memcpy entry points is named.
* Nothing under the package or the headers refers to the oracle (the product never routes through the checker).
"""
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCES = sorted(glob.glob(os.path.join(ROOT, "ullm-project_b200", "csrc", "*")) + glob.glob(os.path.join(ROOT, "include", "*")))


def _lines_outside_tuning(path):
    """Yields (line number, text) of the lines that are compiled without -DULLM_CUDA_TUNING."""
    stack = []  # one entry per open #if: True while the branch in hand is tuning-only
    for no, line in enumerate(open(path, encoding="utf-8", errors="replace"), 1):
        t = line.strip()
        if t.startswith("#ifdef") or t.startswith("#ifndef") or t.startswith("#if "):
            stack.append(t.startswith("#ifdef") and "ULLM_CUDA_TUNING" in t)
            if t.startswith("#ifndef") and "ULLM_CUDA_TUNING" in t:
                stack[-1] = False
            continue
        if t.startswith("#else") and stack:
            stack[-1] = False if stack[-1] else stack[-1]
            continue
        if t.startswith("#endif") and stack:
            stack.pop()
            continue
        if not any(stack):
            yield no, line


def test_the_shipped_library_reads_no_environment_variable():
    assert SOURCES
    for path in SOURCES:
        if os.path.isdir(path) or path.endswith("Makefile"):
            continue
        for no, line in _lines_outside_tuning(path):
            code = line.split("//")[0]
            assert "getenv" not in code, f"{os.path.relpath(path, ROOT)}:{no} reads the environment outside a tuning build"


def test_no_multicast_load_and_no_batched_memcpy_anywhere():
    banned_calls = ["cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync", "cuMemcpy" + "BatchAsync", "cuMemcpy3D" + "BatchAsync"]
    for path in SOURCES + [os.path.join(ROOT, "bench.py"), os.path.join(ROOT, "__graft_entry__.py")]:
        if os.path.isdir(path):
            continue
        text = open(path, encoding="utf-8", errors="replace").read()
        for name in banned_calls:
            assert name not in text, (path, name)
        for m in re.finditer(r"cp\.async\.bulk[^\"\n;]*", text):
            assert "multicast" not in m.group(0), (path, m.group(0))


def test_the_product_never_touches_the_oracle():
    for path in SOURCES + sorted(glob.glob(os.path.join(ROOT, "ullm-project_b200", "ullm_cuda", "*.py"))):
        if os.path.isdir(path):
            continue
        for no, line in enumerate(open(path, encoding="utf-8", errors="replace"), 1):
            code = line.split("//")[0].split("#")[0] if path.endswith(".py") else line.split("//")[0]
            assert not re.search(r"\boracle[/_.]", code) or "oracle" in os.path.basename(path), (path, no, line.strip())
