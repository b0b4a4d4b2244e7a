"""Builds the native libraries in-tree with nvcc / g++ (no torch headers, seconds per file).

    python -m pfeife_b200.csrc.build [--force] [--verbose]

Outputs, next to the package's ``__init__.py``:
  * ``libpfeife_b200_kernels.so`` - every CUDA kernel, compiled for sm_100a only
  * ``libpfeife_b200_host.so``    - host-side C++ (planner evaluator, step executor helpers)

Objects are cached under ``build/`` keyed by source mtime, so rebuilding after a one-file edit
recompiles one file.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
BUILD = PKG.parent / "build" / "pfeife_b200"

KERNEL_LIB = PKG / "libpfeife_b200_kernels.so"
HOST_LIB = PKG / "libpfeife_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
# Approximate division / square root / transcendentals are fine for activations and softmax,
# not for the optimizer update: those two files are bandwidth-bound and keep IEEE arithmetic.
FAST_MATH = ["--use_fast_math"]
PRECISE_SOURCES = {"optim.cu", "dp_fused.cu"}
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(obj: Path, deps: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed:\n{' '.join(cmd)}\n{r.stdout}")
    if verbose and r.stdout.strip():
        print(r.stdout)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> None:
    BUILD.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    nvcc = _nvcc()
    jobs = []
    objs_cu, objs_cpp = [], []
    for src in cu:
        obj = BUILD / (src.stem + ".cu.o")
        objs_cu.append(obj)
        if force or _stale(obj, [src] + headers):
            flags = list(NVCC_FLAGS) + ([] if src.name in PRECISE_SOURCES else FAST_MATH) + \
                (["-Xptxas", "-v"] if ptxas_info else [])
            jobs.append([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    for src in cpp:
        obj = BUILD / (src.stem + ".cpp.o")
        objs_cpp.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append(["g++", *CXX_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    if objs_cu and (force or jobs or _stale(KERNEL_LIB, objs_cu)):
        _run([nvcc, "-shared", "-o", str(KERNEL_LIB), *map(str, objs_cu),
              "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    if objs_cpp and (force or jobs or _stale(HOST_LIB, objs_cpp)):
        _run(["g++", "-shared", "-o", str(HOST_LIB), *map(str, objs_cpp), "-pthread"], verbose)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / smem")
    a = ap.parse_args(argv)
    build(a.force, a.verbose, a.ptxas_info)
    print(f"built {KERNEL_LIB.name}" + (f" and {HOST_LIB.name}" if HOST_LIB.exists() else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
