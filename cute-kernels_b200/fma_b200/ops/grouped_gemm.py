"""grouped_gemm with the reference's call surface (fma/ops/grouped_gemm/__init__.py:11-46)."""

from __future__ import annotations

import torch

from .. import _native
from ..utils import ensure_contiguous
from ._custom_ops import grouped_gemm_op


@ensure_contiguous
def grouped_gemm(
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor | None,
    M_array: torch.Tensor,
    N_array: torch.Tensor,
    K_array: torch.Tensor,
    output_shape: tuple[int, int],
    alpha: float = 1,
    beta: float = 0,
    is_A_transposed: bool = False,
    is_B_transposed: bool = False,
    benchmark: bool = False,
) -> torch.Tensor:
    """Per group g: D_g[M_g,N_g] = A_g . B_g, all matrices packed back to back in flat buffers
    (bf16, fp32 accumulate).  A_g is [M_g,K_g] row-major ([K_g,M_g] if `is_A_transposed`), B_g is
    [K_g,N_g] row-major ([N_g,K_g] if `is_B_transposed`).

    Unlike the reference this wrapper copies M/N/K to the host (one synchronisation) to build
    per-group TMA descriptors; the MoE layer does not go through it.  `benchmark` is ignored.
    """
    assert beta == 0
    assert C is None
    assert alpha == 1
    assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "grouped_gemm runs in bfloat16"
    _native.require_cuda(A, B)

    if isinstance(output_shape, int):
        output_shape = (output_shape,)
    output = torch.empty(*output_shape, device=A.device, dtype=A.dtype)
    grouped_gemm_op(A, B, output, M_array, N_array, K_array, bool(is_A_transposed), bool(is_B_transposed))
    return output
