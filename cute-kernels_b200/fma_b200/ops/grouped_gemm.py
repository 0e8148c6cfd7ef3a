"""grouped_gemm with the reference's call surface (fma/ops/grouped_gemm/__init__.py:11-46)."""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..utils import ensure_contiguous


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

    M = [int(v) for v in M_array.tolist()]
    N = [int(v) for v in N_array.tolist()]
    K = [int(v) for v in K_array.tolist()]
    G = len(M)
    assert len(N) == G and len(K) == G
    assert sum(m * k for m, k in zip(M, K)) <= A.numel(), "A is smaller than the packed operands"
    assert sum(n * k for n, k in zip(N, K)) <= B.numel(), "B is smaller than the packed operands"
    assert sum(m * n for m, n in zip(M, N)) <= output.numel(), "output_shape is smaller than the packed results"

    arr_t = ctypes.c_uint32 * G
    total_mtiles = sum((m + 127) // 128 for m in M)
    nbytes = _native.lib().fma_b200_grouped_gemm_workspace_bytes(G, total_mtiles)
    workspace = torch.empty(max(nbytes, 128) + 128, dtype=torch.uint8, device=A.device)
    offset = (-workspace.data_ptr()) % 128
    ws_ptr = ctypes.c_void_p(workspace.data_ptr() + offset)
    with torch.cuda.device(A.device):
        _native.call(
            "fma_b200_grouped_gemm",
            _native.ptr(A), _native.ptr(B), _native.ptr(output),
            ctypes.cast(arr_t(*M), ctypes.c_void_p), ctypes.cast(arr_t(*N), ctypes.c_void_p),
            ctypes.cast(arr_t(*K), ctypes.c_void_p),
            G, int(is_A_transposed), int(is_B_transposed), ws_ptr, nbytes, _native.stream_ptr(A.device),
        )  # fmt: skip
    # the workspace is read by the kernel after this call returns: keep it alive on this stream
    workspace.record_stream(torch.cuda.current_stream(A.device))
    return output
