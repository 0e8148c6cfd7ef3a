"""Loads the reference project's own grouped GEMM (built by baseline/build_reference_gemm.py into
baseline/_ref/) and calls it through its stock entry point grouped_gemm_cuda
(fma/ops/grouped_gemm/cuda_implementation/ops.cpp:7-20; kernel.cu:354-388).  Used by bench.py's
`reference_gpu` block and by tests/test_gpu_reference_gemm.py; single-GPU only."""

from __future__ import annotations

import importlib.util
from pathlib import Path

import torch

MODULE = "fma_ref_grouped_gemm"
_PATH = Path(__file__).resolve().parent / "_ref" / f"{MODULE}.so"
_module = None


def available() -> tuple[bool, str]:
    if not _PATH.exists():
        return False, f"{_PATH.name} has not been built (python baseline/build_reference_gemm.py <reference>)"
    if not torch.cuda.is_available():
        return False, "no CUDA device"
    return True, ""


def load():
    global _module
    if _module is None:
        spec = importlib.util.spec_from_file_location(MODULE, _PATH)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _module = mod
    return _module


def grouped_gemm(A, B, M_array, N_array, K_array, output_shape, is_A_transposed=False, is_B_transposed=False):
    """The reference's grouped_gemm with C=None, alpha=1, beta=0 (fma/ops/grouped_gemm/__init__.py:11-46)."""
    out = torch.empty(*output_shape, device=A.device, dtype=A.dtype)
    load().grouped_gemm_cuda(A, B, None, out, M_array, N_array, K_array, is_A_transposed, is_B_transposed, 1.0, 0.0,
                             False)
    return out
