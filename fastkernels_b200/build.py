"""Build libfk_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m fastkernels_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects and the library are written next to
the sources (git-ignored); nothing is installed outside the package directory.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfk_b200.so"
SOURCES = ["fk_host.cu", "fk_elementwise.cu", "fk_attn.cu", "fk_gemm.cu", "fk_comm.cu",
           "fk_prefill.cu", "fk_gemm_large.cu", "fk_block.cu"]
HEADERS = [CSRC / "fk_common.cuh", CSRC / "fk_tcgen05.cuh", CSRC / "fk_rowops.cuh",
           CSRC / "fk_gemm_shared.cuh", PKG.parent / "include" / "fk_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    objs = [s.with_suffix(".o") for s in srcs]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _stale(o, [s, *HEADERS])]
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for out in ex.map(lambda so: _compile(so[0], so[1], verbose), todo):
                if verbose and out.strip():
                    print(out, file=sys.stderr)
    if force or todo or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
