"""swiglu / swiglu_packed with the reference's call surface (fma/ops/swiglu/__init__.py:97-164)."""

from __future__ import annotations

import torch

from .. import _native
from ..kernel_backend import KernelBackend
from ._custom_ops import (
    swiglu_backward_op,
    swiglu_forward_op,
    swiglu_packed_backward_op,
    swiglu_packed_forward_op,
)


def _as_rows(t: torch.Tensor) -> torch.Tensor:
    """Returns `t` or a contiguous copy such that it is [rows, cols] with unit column stride and a
    single row pitch (the two halves of a packed last dimension qualify without a copy)."""
    if t.dim() >= 1 and t.stride(-1) == 1:
        if t.dim() <= 2:
            return t
        # leading dims must collapse onto one pitch
        pitch = t.stride(-2)
        ok = True
        expect = pitch * t.size(-2)
        for d in range(t.dim() - 3, -1, -1):
            if t.size(d) != 1 and t.stride(d) != expect:
                ok = False
                break
            expect *= t.size(d)
        if ok:
            return t
    return t.contiguous()


def _forward(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor) -> None:
    swiglu_forward_op(gate, up, out)


def _backward(gate, up, dy, gate_grad, up_grad) -> None:
    swiglu_backward_op(gate, up, dy, gate_grad, up_grad)


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        assert gate.size() == up.size(), "tensors gate and up should have same shape"
        assert gate.dtype == up.dtype, "tensors gate and up should have same dtype"
        _native.require_cuda(gate, up)
        gate, up = _as_rows(gate), _as_rows(up)
        out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
        _forward(gate, up, out)
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, output_grad: torch.Tensor):
        gate, up = ctx.saved_tensors
        output_grad = output_grad.contiguous()
        gate_grad = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
        up_grad = torch.empty(up.shape, dtype=up.dtype, device=up.device)
        _backward(gate, up, output_grad, gate_grad, up_grad)
        return gate_grad, up_grad


class _SwigluPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        _native.require_cuda(x)
        assert x.size(-1) % 2 == 0
        x = x.contiguous()  # first half of the last dimension is `up`, second half is `gate`
        out = torch.empty(*x.shape[:-1], x.size(-1) // 2, dtype=x.dtype, device=x.device)
        swiglu_packed_forward_op(x, out)
        ctx.save_for_backward(x)
        return out

    @staticmethod
    def backward(ctx, output_grad: torch.Tensor):
        (x,) = ctx.saved_tensors
        output_grad = output_grad.contiguous()
        x_grad = torch.empty_like(x)
        swiglu_packed_backward_op(x, output_grad, x_grad)
        return x_grad


def swiglu(
    gate: torch.Tensor,
    up: torch.Tensor,
    *,
    kernel_backend_forward: KernelBackend = KernelBackend.cuda,
    kernel_backend_backward: KernelBackend = KernelBackend.cuda,
) -> torch.Tensor:
    """`up * gate * sigmoid(gate)`, computed in fp32 and cast back.  The backend arguments are
    accepted for compatibility and select nothing."""
    return _Swiglu.apply(gate, up)


def swiglu_packed(
    x: torch.Tensor,
    *,
    kernel_backend_forward: KernelBackend = KernelBackend.triton,
    kernel_backend_backward: KernelBackend = KernelBackend.triton,
) -> torch.Tensor:
    """SwiGLU of a packed tensor: `up, gate = x.chunk(2, dim=-1)`.  Inside `MoE` this function is
    recognised and runs in the epilogue of the up-projection GEMM instead."""
    return _SwigluPacked.apply(x)
