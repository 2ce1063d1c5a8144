"""Build libfk_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m fastkernels_b200.build [--force] [--verbose]
    python -m fastkernels_b200.build --define FK_GEMM_TRACE --define FK_BLOCK_TRACE   (diagnostic copy)

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


def _compile(src: Path, obj: Path, verbose: bool, defines=()) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False, defines=(), out: Path | None = None) -> Path:
    """Default: the library proper, objects next to the sources.  With `defines`
    (e.g. FK_GEMM_TRACE, FK_BLOCK_TRACE: per-CTA time stamps for
    `microbench timeline`) a diagnostic copy is built into `out`'s directory and
    loaded by setting FK_B200_LIB to it."""
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    lib = LIB
    if defines or out is not None:
        lib = Path(out) if out is not None else PKG.parent / "build" / "libfk_b200_diag.so"
        # objects of a diagnostic copy live beside it, in a folder of its own: two
        # copies built with different defines must not pick up each other's objects
        objdir = lib.parent / (lib.stem + "_objs")
        objdir.mkdir(parents=True, exist_ok=True)
        objs = [objdir / (s.stem + ".o") for s in srcs]
    else:
        objs = [s.with_suffix(".o") for s in srcs]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _stale(o, [s, *HEADERS])]
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for res in ex.map(lambda so: _compile(so[0], so[1], verbose, defines), todo):
                if verbose and res.strip():
                    print(res, file=sys.stderr)
    if force or todo or _stale(lib, objs):
        cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[],
                    help="preprocessor switch for a diagnostic build (repeatable)")
    ap.add_argument("--out", default=None, help="library path of a diagnostic build")
    a = ap.parse_args()
    print(build(a.force, a.verbose, tuple(a.define), a.out))
