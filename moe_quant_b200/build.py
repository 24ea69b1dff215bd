"""Builds libmoequant_sm100.so in-tree with nvcc for sm_100a.

    python -m moe_quant_b200.build

nvcc cross-compiles without a GPU.  Objects go to moe_quant_b200/csrc/build/ and
the library next to this file, so a source snapshot carries the binary with it.
"""
from __future__ import annotations

import concurrent.futures
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmoequant_sm100.so")
SOURCES = ["api.cu", "pack.cu", "prepare.cu", "gemm_simt.cu", "hinv.cu", "sweep.cu", "umma_gemm.cu", "profile.cu", "metrics.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA engine cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _includes(path: str, dirs, seen=None):
    """`path` and every file it includes with quotes, recursively (searched in `dirs`): a source
    is recompiled when one of these is newer than its object.  The row-per-thread sweep kernels
    take minutes to compile, so a change elsewhere should not rebuild them."""
    seen = seen if seen is not None else []
    if path in seen:
        return seen
    seen.append(path)
    with open(path) as f:
        names = re.findall(r'^\s*#\s*include\s+"([^"]+)"', f.read(), flags=re.M)
    for name in names:
        for d in dirs:
            cand = os.path.join(d, name)
            if os.path.exists(cand):
                _includes(cand, dirs, seen)
                break
    return seen


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    inc = os.path.join(os.path.dirname(HERE), "include")

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if force or _stale(obj, _includes(path, (CSRC, inc))):
            cmd = [nvcc, *FLAGS, "-c", path, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            log = os.path.join(objdir, src + ".log")
            with open(log, "w") as f:
                f.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, len(SOURCES))) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    if force or _stale(OUT, objs):
        cmd = [nvcc, "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
