"""Builds the reference project's own sm_100 grouped GEMM (its CUTLASS kernel, unmodified, compiled from
the sources where they lie) into baseline/_ref/, so that bench.py --workload gemm_vs_reference can time it
next to this library's grouped GEMMs on one GPU.

    python baseline/build_reference_gemm.py /path/to/reference

The reference builds this file at run time with torch.utils.cpp_extension.load
(fma/jit.py:22-52) against its `cutlass` submodule, which its snapshot leaves empty; this script
compiles the same two sources (fma/ops/grouped_gemm/cuda_implementation/kernel.cu and ops.cpp) with the
reference's flags (-O3 -lineinfo) against the CUTLASS headers found in the Python environment, for
sm_100a (the kernel's tcgen05 instructions need the architecture-specific target).  Nothing is copied
into the repository: outputs are an object file and the extension module under baseline/_ref/, which is
not under version control.  The kernel's CUTLASS collective broadcasts operand tiles to the CTAs of a
cluster, so it may only be run by single-GPU jobs on memory of that GPU.
"""

from __future__ import annotations

import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
OUT = ROOT / "_ref"
MODULE = "fma_ref_grouped_gemm"


def cutlass_root() -> Path | None:
    import importlib.util

    for pkg in ("flashinfer", "tilelang"):
        spec = importlib.util.find_spec(pkg)
        if spec is None or not spec.submodule_search_locations:
            continue
        base = Path(list(spec.submodule_search_locations)[0])
        for cand in (base / "data" / "cutlass", base / "3rdparty" / "cutlass"):
            if (cand / "include" / "cutlass" / "cutlass.h").exists() and (cand / "tools" / "util" / "include").exists():
                return cand
    return None


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    ref = Path(sys.argv[1]).resolve()
    src_dir = ref / "fma" / "ops" / "grouped_gemm" / "cuda_implementation"
    if not (src_dir / "kernel.cu").exists():
        print(f"{src_dir}/kernel.cu not found")
        return 2
    cutlass = cutlass_root()
    if cutlass is None:
        print("no CUTLASS header tree with tools/util/include found in the Python environment")
        return 3
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    OUT.mkdir(parents=True, exist_ok=True)
    incs = [str(ref / "fma"), str(cutlass / "include"), str(cutlass / "tools" / "util" / "include"),
            sysconfig.get_paths()["include"], *include_paths("cuda")]  # fmt: skip
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]  # fmt: skip
    inc_flags = [f"-I{p}" for p in incs]
    log = OUT / "build.log"
    steps = [
        ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
         "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC", *defs, *inc_flags, "-c",
         str(src_dir / "kernel.cu"), "-o", str(OUT / "kernel.o")],
        ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc_flags, "-c", str(src_dir / "ops.cpp"), "-o", str(OUT / "ops.o")],
        ["g++", "-shared", str(OUT / "kernel.o"), str(OUT / "ops.o"), "-o", str(OUT / f"{MODULE}.so"),
         *[f"-L{p}" for p in library_paths("cuda")], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
         "-ltorch_python", "-lcudart"],
    ]  # fmt: skip
    with open(log, "w") as f:
        f.write(f"CUTLASS headers: {cutlass}\n")
        for cmd in steps:
            f.write("$ " + " ".join(cmd) + "\n")
            f.flush()
            res = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT)
            if res.returncode != 0:
                print(f"step failed ({cmd[0]}), see {log}")
                return 1
    print(OUT / f"{MODULE}.so")
    return 0


if __name__ == "__main__":
    sys.exit(main())
