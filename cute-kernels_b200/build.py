"""Builds libfma_b200.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

Usage:  python cute-kernels_b200/build.py [--force] [--verbose]

The library is compiled for sm_100a only (explicit -gencode; the -arch=sm_100a shorthand also
emits generic compute_100 PTX, which rejects tcgen05).  Objects and the .so stay next to the
sources; nothing is installed outside the tree.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "fma_b200" / "_lib"
LIB_PATH = OUT_DIR / "libfma_b200.so"
HEADER = ROOT.parent / "include" / "fma_b200.h"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return nvcc


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every csrc/*.cu and links libfma_b200.so; returns its path."""
    nvcc = _nvcc()
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [HEADER, Path(__file__)]
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))

    if force or _stale(LIB_PATH, objects):
        # Export only the fma_b200_* entry points (the driver entry point for tensor maps is
        # resolved at run time through cudaGetDriverEntryPoint, so libcuda is not linked).
        vers = OUT_DIR / "exports.map"
        vers.write_text("{ global: fma_b200_*; local: *; };\n")
        cmd = [
            nvcc,
            "-shared",
            "-gencode",
            "arch=compute_100a,code=sm_100a",
            "-o",
            str(LIB_PATH),
            *[str(o) for o in objects],
            "-Xlinker",
            f"--version-script={vers}",
        ]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libfma_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build_library(force=args.force, verbose=args.verbose))
