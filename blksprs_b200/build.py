"""Builds the C-ABI shared library ``libblksprs_b200.so`` in-tree with nvcc for sm_100a.

Run as ``python -m blksprs_b200.build`` (add ``--force`` to rebuild everything).
The library is a plain ``extern "C"`` shared object (no torch types); the Python
package loads it with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "lib"
LIB_PATH = OUT_DIR / "libblksprs_b200.so"
SOURCES = ["capi.cu", "lut.cu", "plan_panel.cu", "matmul_mma.cu", "matmul_umma.cu", "conversion.cu", "softmax.cu",
           "linear.cu"]
HEADERS = [CSRC / "common.cuh", CSRC / "umma_common.cuh", PKG_DIR.parent / "include" / "blksprs_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    if cand.exists():
        return str(cand)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    (obj.with_suffix(".ptxas.txt")).write_text(res.stderr)
    if verbose:
        print(res.stderr, file=sys.stderr)
    return src.name


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every ``csrc/*.cu`` for sm_100a and links ``lib/libblksprs_b200.so``."""
    nvcc = find_nvcc()
    OUT_DIR.mkdir(exist_ok=True)
    jobs = []
    objs = []
    for name in SOURCES:
        src = CSRC / name
        obj = OUT_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *HEADERS]):
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs))
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
