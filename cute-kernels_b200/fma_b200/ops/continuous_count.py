"""continuous_count with the reference's call surface (fma/ops/continuous_count/__init__.py:11-43)."""

from __future__ import annotations

import torch

from .. import _native
from ..kernel_backend import KernelBackend

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, size: int) -> torch.Tensor:
    """Per-device scratch for the block partials; its ticket word starts at zero and every call
    leaves it at zero, so it is allocated once and reused by later calls on the same stream order."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), size)
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = _native.lib().fma_b200_continuous_count_workspace_bytes(size)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


@torch.no_grad()
def continuous_count(
    x: torch.Tensor, size: int, *, kernel_backend: KernelBackend = KernelBackend.cuda, _variant: int | None = None
) -> torch.Tensor:
    """Counts the occurrences of the values [0, size) in the 1-D int32/int64 tensor `x`.

    Values outside the range are ignored.  Returns a uint32 tensor of `size` elements, like the
    reference.  `kernel_backend` is accepted for compatibility and selects nothing.
    """
    if size == 1:
        return torch.tensor([x.numel()], dtype=torch.uint32, device=x.device)

    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in [torch.int32, torch.long]
    _native.require_cuda(x)
    x = x.contiguous()
    if x.data_ptr() % 16 != 0:  # the kernel reads 128-bit vectors
        x = x.clone()

    output = torch.empty(size, dtype=torch.uint32, device=x.device)
    ws = _workspace(x.device, size)
    args = (_native.ptr(x), x.element_size(), x.numel(), size, _native.ptr(output), _native.ptr(ws), ws.numel())
    with torch.cuda.device(x.device):
        if _variant is None:  # the library picks the shared-memory scheme from `size`
            _native.call("fma_b200_continuous_count", *args, _native.stream_ptr(x.device))
        else:  # measurement hook: force one scheme
            _native.call("fma_b200_continuous_count_variant", *args, _variant, _native.stream_ptr(x.device))
    return output
