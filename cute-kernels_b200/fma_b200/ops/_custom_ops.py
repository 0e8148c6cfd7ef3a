"""torch.library custom ops around the C-ABI kernels of the op surface, in the reference's style:
out-parameter ops that return None and declare what they mutate (e.g. the reference's
fma/ops/continuous_count/cuda_implementation/__init__.py:12-16), which is what lets
torch.compile(fullgraph=True) trace code that calls them.  The bodies are opaque to the compiler; they
hold everything that needs real pointers (alignment fixes, workspaces, the ctypes calls)."""

from __future__ import annotations

import ctypes

import torch

from .. import _native

LIBRARY_NAME = "flash_model_architectures_b200"

_count_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _count_workspace(device: torch.device, size: int) -> torch.Tensor:
    """Per-device scratch (ticket + accumulators), zero-filled once; every call leaves it zero-filled."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), size)
    ws = _count_workspaces.get(key)
    if ws is None:
        nbytes = _native.lib().fma_b200_continuous_count_workspace_bytes(size)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _count_workspaces[key] = ws
    return ws


@torch.library.custom_op(f"{LIBRARY_NAME}::continuous_count", mutates_args={"output"})
def continuous_count_op(x: torch.Tensor, output: torch.Tensor, size: int, variant: int) -> None:
    _native.require_cuda(x, output)
    x = x.contiguous()
    if x.data_ptr() % 16 != 0:  # the kernel reads 128-bit vectors
        x = x.clone()
    ws = _count_workspace(x.device, size)
    args = (_native.ptr(x), x.element_size(), x.numel(), size, _native.ptr(output), _native.ptr(ws), ws.numel())
    with torch.cuda.device(x.device):
        if variant < 0:  # the library picks the shared-memory scheme
            _native.call("fma_b200_continuous_count", *args, _native.stream_ptr(x.device))
        else:  # measurement hook: force one scheme
            _native.call("fma_b200_continuous_count_variant", *args, variant, _native.stream_ptr(x.device))


def _rows_cols(t: torch.Tensor) -> tuple[int, int]:
    cols = t.size(-1)
    return (t.numel() // cols if cols else 0), cols


def _pitch(t: torch.Tensor) -> int:
    return t.size(0) if t.dim() == 1 else t.stride(-2)


@torch.library.custom_op(f"{LIBRARY_NAME}::swiglu_forward", mutates_args={"output"})
def swiglu_forward_op(gate: torch.Tensor, up: torch.Tensor, output: torch.Tensor) -> None:
    _native.require_cuda(gate, up, output)
    rows, cols = _rows_cols(output)
    with torch.cuda.device(output.device):
        _native.call(
            "fma_b200_swiglu_forward",
            _native.ptr(gate), _pitch(gate), _native.ptr(up), _pitch(up), _native.ptr(output), _pitch(output),
            _native.dtype_code(output.dtype), rows, cols, _native.stream_ptr(output.device),
        )  # fmt: skip


@torch.library.custom_op(f"{LIBRARY_NAME}::swiglu_backward", mutates_args={"gate_grad", "up_grad"})
def swiglu_backward_op(
    gate: torch.Tensor, up: torch.Tensor, output_grad: torch.Tensor, gate_grad: torch.Tensor, up_grad: torch.Tensor
) -> None:
    _native.require_cuda(gate, up, output_grad)
    rows, cols = _rows_cols(output_grad)
    with torch.cuda.device(output_grad.device):
        _native.call(
            "fma_b200_swiglu_backward",
            _native.ptr(gate), _pitch(gate), _native.ptr(up), _pitch(up), _native.ptr(output_grad), _pitch(output_grad),
            _native.ptr(gate_grad), _pitch(gate_grad), _native.ptr(up_grad), _pitch(up_grad),
            _native.dtype_code(output_grad.dtype), rows, cols, _native.stream_ptr(output_grad.device),
        )  # fmt: skip


@torch.library.custom_op(f"{LIBRARY_NAME}::swiglu_packed_forward", mutates_args={"output"})
def swiglu_packed_forward_op(x: torch.Tensor, output: torch.Tensor) -> None:
    """x is contiguous [..., 2c]: the first half of the last dimension is `up`, the second `gate`."""
    up, gate = x.chunk(2, dim=-1)
    swiglu_forward_op(gate, up, output)


@torch.library.custom_op(f"{LIBRARY_NAME}::swiglu_packed_backward", mutates_args={"x_grad"})
def swiglu_packed_backward_op(x: torch.Tensor, output_grad: torch.Tensor, x_grad: torch.Tensor) -> None:
    up, gate = x.chunk(2, dim=-1)
    up_grad, gate_grad = x_grad.chunk(2, dim=-1)
    swiglu_backward_op(gate, up, output_grad, gate_grad, up_grad)


@torch.library.custom_op(f"{LIBRARY_NAME}::grouped_gemm", mutates_args={"output"})
def grouped_gemm_op(
    A: torch.Tensor,
    B: torch.Tensor,
    output: torch.Tensor,
    M_array: torch.Tensor,
    N_array: torch.Tensor,
    K_array: torch.Tensor,
    is_A_transposed: bool,
    is_B_transposed: bool,
) -> None:
    _native.require_cuda(A, B, output)
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
    ws_ptr = ctypes.c_void_p(workspace.data_ptr() + (-workspace.data_ptr()) % 128)
    with torch.cuda.device(A.device):
        _native.call(
            "fma_b200_grouped_gemm",
            _native.ptr(A), _native.ptr(B), _native.ptr(output),
            ctypes.cast(arr_t(*M), ctypes.c_void_p), ctypes.cast(arr_t(*N), ctypes.c_void_p),
            ctypes.cast(arr_t(*K), ctypes.c_void_p),
            G, int(is_A_transposed), int(is_B_transposed), ws_ptr, nbytes, _native.stream_ptr(A.device),
        )  # fmt: skip
