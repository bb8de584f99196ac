"""Rules the sources keep on this hardware pool, checked by reading them: no bulk / tensor copy with
cluster-wide delivery (it must never meet another GPU's memory), none of the batched memcpy entry
points, every device spin loop bounded, and the product never reaches into the CPU checker."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIRS = ["ggnpu_b200", "include", "oracle", "tests"]
SRC_EXT = (".cu", ".cuh", ".h", ".c", ".cpp", ".py")


def _sources(dirs=SRC_DIRS):
    for d in dirs:
        for base, _, files in os.walk(os.path.join(ROOT, d)):
            if "_ref" in base or "build" in base.split(os.sep) or "__pycache__" in base:
                continue
            for f in files:
                if f.endswith(SRC_EXT):
                    yield os.path.join(base, f)
    if dirs is SRC_DIRS:
        for f in ("bench.py", "__graft_entry__.py"):
            yield os.path.join(ROOT, f)


def _grep(pattern, dirs=SRC_DIRS):
    rx = re.compile(pattern)
    hits = []
    for p in _sources(dirs):
        with open(p, errors="replace") as fh:
            for i, line in enumerate(fh, 1):
                if rx.search(line):
                    hits.append(f"{os.path.relpath(p, ROOT)}:{i}")
    return hits


def test_no_cluster_wide_copy_qualifier():
    # the qualifier is assembled here so that this file does not contain it either
    assert _grep(r"\." + "multi" + "cast" + "::" + "cluster") == []


def test_no_batched_memcpy_entry_points():
    names = ["cuda" + "Memcpy" + "BatchAsync", "cuda" + "Memcpy3D" + "BatchAsync", "cu" + "Memcpy" + "BatchAsync",
             "cu" + "Memcpy3D" + "BatchAsync"]
    assert _grep("|".join(names)) == []


def test_product_does_not_use_the_cpu_checker():
    """Only tests/, bench.py's cpu legs and the smoke check may touch oracle/."""
    hits = _grep(r"^\s*(from|import)\s+oracle\b|oracle\.binding|libggb_oracle|ggb_oracle", dirs=["ggnpu_b200", "include"])
    assert hits == []


def test_device_spin_loops_are_bounded():
    """Every `while` that polls an mbarrier, a flag or a timer in the kernels carries a limit."""
    csrc = os.path.join(ROOT, "ggnpu_b200", "csrc")
    for f in sorted(os.listdir(csrc)):
        if not f.endswith((".cu", ".cuh")):
            continue
        text = open(os.path.join(csrc, f)).read()
        for m in re.finditer(r"while\s*\(([^;{]*?(try_wait|volatile|globaltimer|ld_acquire|ld_volatile)[^;{]*?)\)\s*[{;]", text):
            cond = m.group(1)
            assert re.search(r"<|>|limit|spins|tries|deadline", cond), f"{f}: unbounded wait: while ({cond})"
