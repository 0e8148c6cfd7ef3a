"""continuous_count with the reference's call surface (fma/ops/continuous_count/__init__.py:11-43)."""

from __future__ import annotations

import torch

from .. import _native
from ..kernel_backend import KernelBackend
from ._custom_ops import continuous_count_op

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

    output = torch.empty(size, dtype=torch.uint32, device=x.device)
    continuous_count_op(x, output, size, -1 if _variant is None else _variant)
    return output
