"""Build libggb200.so (the CUDA kernels and the C ABI) in-tree with nvcc for sm_100a.

    python -m ggnpu_b200.build [--force] [--verbose-ptxas]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically,
so it only needs the NVIDIA driver at run time.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libggb200.so")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
         "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "ggb200.h"),
                                                                 os.path.join(HERE, "iq_tables.py")]
    return max(os.path.getmtime(f) for f in files)


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _deps_mtime():
        return OUT
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    # codebooks of the grid-coded formats, generated from the gguf package (absent: built without them)
    from .iq_tables import write_include
    if not write_include(os.path.join(OBJ, "ggb_iq_grids.inc")):
        sys.stderr.write("ggnpu_b200.build: gguf package not found, IQ1/IQ2/IQ3 formats left out\n")
    extra += ["-I", OBJ]
    extra += os.environ.get("GGB_NVCC_FLAGS", "").split()        # e.g. -DGGB_STEP_TRACE (time stamps in the decode-step kernel)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [NVCC, *ARCH, *FLAGS, *extra, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose_ptxas:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [NVCC, *ARCH, "-shared", "-o", OUT, *objs, "-Xcompiler", "-fPIC", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv))
