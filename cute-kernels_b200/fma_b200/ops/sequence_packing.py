"""pack_sequence / unpack_sequence with the reference's call surface
(fma/ops/sequence_packing/__init__.py:156-245): padded batches [B, S, ...] <-> packed token lists
[total, ...] described by cu_seqlens.  One HBM-bound copy kernel each way; unpacking writes the padding as
zeros in the same pass.  `kernel_backend_*` arguments are accepted for compatibility and select nothing."""

from __future__ import annotations

import torch

from .. import _native
from ..kernel_backend import KernelBackend
from ._custom_ops import LIBRARY_NAME


@torch.library.custom_op(f"{LIBRARY_NAME}::pack_unpack_sequence", mutates_args={"output"})
def pack_unpack_sequence_op(x: torch.Tensor, output: torch.Tensor, cu_seqlens: torch.Tensor, pad_left: bool,
                            pack: bool) -> None:
    """pack: x [B, S, ...] -> output [total, ...]; unpack: x [total, ...] -> output [B, S, ...] (fully written)."""
    _native.require_cuda(x, output, cu_seqlens)
    x = x.contiguous()
    padded, packed = (x, output) if pack else (output, x)
    B, S = padded.size(0), padded.size(1)
    total = packed.size(0)
    row_bytes = (padded.numel() // max(B * S, 1)) * padded.element_size() if B * S else packed[0].numel() * packed.element_size()
    assert cu_seqlens.numel() == B + 1 and cu_seqlens.is_contiguous()
    assert cu_seqlens.dtype in (torch.uint32, torch.int32, torch.int64)
    name = "fma_b200_pack_sequence" if pack else "fma_b200_unpack_sequence"
    with torch.cuda.device(x.device):
        _native.call(name, _native.ptr(x), _native.ptr(output), _native.ptr(cu_seqlens), cu_seqlens.element_size(), B, S,
                     total, row_bytes, int(pad_left), _native.stream_ptr(x.device))  # fmt: skip


def _check_side(padding_side: str) -> bool:
    if padding_side not in ("left", "right"):
        raise ValueError(f"unexpected padding_side ({padding_side})")
    return padding_side == "left"


class _PackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu_seqlens, output_shape, padding_side):
        assert x.dim() >= 2 and x.size(0) == cu_seqlens.size(0) - 1
        ctx.save_for_backward(cu_seqlens)
        ctx.padding_side, ctx.x_shape = padding_side, x.size()
        output = torch.empty(output_shape, device=x.device, dtype=x.dtype)
        pack_unpack_sequence_op(x, output, cu_seqlens, _check_side(padding_side), True)
        return output

    @staticmethod
    def backward(ctx, output_grad):
        x_grad = torch.empty(ctx.x_shape, device=output_grad.device, dtype=output_grad.dtype)
        pack_unpack_sequence_op(output_grad, x_grad, ctx.saved_tensors[0], _check_side(ctx.padding_side), False)
        return x_grad, None, None, None


class _UnpackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu_seqlens, output_shape, padding_side):
        assert x.dim() >= 2 and output_shape[0] == cu_seqlens.size(0) - 1
        assert tuple(output_shape[2:]) == tuple(x.size()[1:])
        ctx.save_for_backward(cu_seqlens)
        ctx.padding_side, ctx.x_shape = padding_side, x.size()
        output = torch.empty(tuple(output_shape), device=x.device, dtype=x.dtype)
        pack_unpack_sequence_op(x, output, cu_seqlens, _check_side(padding_side), False)
        return output

    @staticmethod
    def backward(ctx, output_grad):
        x_grad = torch.empty(ctx.x_shape, device=output_grad.device, dtype=output_grad.dtype)
        pack_unpack_sequence_op(output_grad, x_grad, ctx.saved_tensors[0], _check_side(ctx.padding_side), True)
        return x_grad, None, None, None


def pack_sequence(
    inputs: torch.Tensor | list[torch.Tensor],
    cu_seqlens: torch.Tensor,
    output_shape: tuple[int] | None = None,
    padding_side: str = "left",
    *,
    kernel_backend_forward: KernelBackend = KernelBackend.cuda,
    kernel_backend_backward: KernelBackend = KernelBackend.cuda,
) -> torch.Tensor | list[torch.Tensor]:
    is_list = isinstance(inputs, (list, tuple))
    if not is_list:
        inputs = [inputs]
    outputs = []
    total = None
    for x in inputs:
        shape = output_shape
        if shape is None:
            if total is None:  # one host read of the token count for all tensors, as the reference does
                total = int(cu_seqlens[-1].item())
            shape = (total, *x.size()[2:])
        outputs.append(_PackSequence.apply(x, cu_seqlens, tuple(shape), padding_side))
    return outputs if is_list else outputs[0]


def unpack_sequence(
    inputs: torch.Tensor | list[torch.Tensor],
    cu_seqlens: torch.Tensor,
    output_shape: tuple[int],
    padding_side: str = "left",
    *,
    kernel_backend_forward: KernelBackend = KernelBackend.cuda,
    kernel_backend_backward: KernelBackend = KernelBackend.cuda,
) -> torch.Tensor | list[torch.Tensor]:
    is_list = isinstance(inputs, (list, tuple))
    if not is_list:
        inputs = [inputs]
    outputs = [_UnpackSequence.apply(x, cu_seqlens, tuple(output_shape), padding_side) for x in inputs]
    return outputs if is_list else outputs[0]
