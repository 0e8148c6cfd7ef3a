"""The MoE layer as torch.library custom ops, so that torch.compile(fullgraph=True) can trace
`MoE.forward` (the reference compiles its MoE in tests/modules/moe_test.py:97-98).  Two ops with
registered autograd: the router's top-k + softmax, and the SwiGLU experts from token scatter to weighted
combine.  Their bodies are opaque to the compiler and run the same kernels, in the same order, as the
eager path (`moe._FusedSwigluExperts`); tensors that the backward needs are extra outputs of the forward
op.  All shapes follow from the input shapes alone (rows_cap does not depend on the routing), which is
what the fake implementations rely on."""

from __future__ import annotations

import torch

from ..ops._custom_ops import LIBRARY_NAME
from . import _kernels as K


def _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k: int, row_align: int, expert_count=None):
    return K.RowMaps(expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert, slot_of_row.size(0),
                     pad_offsets.numel() - 1, top_k, row_align)  # fmt: skip


# ---- router: top-k + softmax ---------------------------------------------------------------------
@torch.library.custom_op(f"{LIBRARY_NAME}::moe_route", mutates_args=())
def moe_route(logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (weights, selected, workspace); the workspace carries the expert sort's first pass to
    moe_swiglu_experts."""
    with torch.cuda.device(logits.device):
        return K.router_topk_softmax_routed(logits, top_k)


@moe_route.register_fake
def _(logits, top_k):
    T, E = logits.shape
    return (logits.new_empty(T, top_k), logits.new_empty((T, top_k), dtype=torch.int64),
            logits.new_empty(K.sort_workspace_bytes(T * top_k, E), dtype=torch.uint8))  # fmt: skip


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_route_backward", mutates_args=())
def moe_route_backward(weights: torch.Tensor, d_weights: torch.Tensor, selected: torch.Tensor,
                       num_experts: int) -> torch.Tensor:  # fmt: skip
    with torch.cuda.device(weights.device):
        return K.router_topk_softmax_backward(weights, d_weights, selected, num_experts)


@moe_route_backward.register_fake
def _(weights, d_weights, selected, num_experts):
    return weights.new_empty(weights.size(0), num_experts)


def _route_setup(ctx, inputs, output):
    logits, _ = inputs
    weights, selected, _workspace = output
    ctx.save_for_backward(weights, selected)
    ctx.num_experts = logits.size(1)


def _route_backward(ctx, d_weights, _d_selected, _d_workspace):
    weights, selected = ctx.saved_tensors
    return moe_route_backward(weights, d_weights.contiguous(), selected, ctx.num_experts), None


torch.library.register_autograd(f"{LIBRARY_NAME}::moe_route", _route_backward, setup_context=_route_setup)


# ---- experts: scatter -> up projection + SwiGLU -> down projection -> weighted combine ------------
@torch.library.custom_op(f"{LIBRARY_NAME}::moe_swiglu_experts", mutates_args=())
def moe_swiglu_experts(
    x: torch.Tensor, weights: torch.Tensor, selected: torch.Tensor, route_workspace: torch.Tensor, w_fc: torch.Tensor,
    w_proj: torch.Tensor, row_align: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor]:  # fmt: skip
    """Returns (y, xg, pre, act, out, expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert)."""
    with torch.cuda.device(x.device):
        x, weights, w_fc, w_proj = x.contiguous(), weights.contiguous(), w_fc.contiguous(), w_proj.contiguous()
        maps = K.moe_sort(selected, w_fc.size(0), row_align=row_align, routed_workspace=route_workspace)
        xg = K.scatter(x, maps)
        pre, act = K.gemm_forward_swiglu(xg, w_fc, maps.mtile_expert, keep_pre=True, row_align=row_align)
        out = K.gemm_forward(act, w_proj, maps.mtile_expert, row_align)
        y = K.combine(out, weights, maps, x.size(0))
    return (y, xg, pre, act, out, maps.expert_count, maps.pad_offsets, maps.row_of_slot, maps.slot_of_row,
            maps.mtile_expert)  # fmt: skip


@moe_swiglu_experts.register_fake
def _(x, weights, selected, route_workspace, w_fc, w_proj, row_align):
    T, H = x.shape
    E, two_i, _ = w_fc.shape
    R = selected.numel()
    cap = K.rows_cap(R, E, row_align)
    i32 = lambda *shape: x.new_empty(shape, dtype=torch.int32)  # noqa: E731
    return (x.new_empty(T, H), x.new_empty(cap, H), x.new_empty(cap, two_i), x.new_empty(cap, two_i // 2),
            x.new_empty(cap, H), x.new_empty((E,), dtype=torch.uint32), i32(E + 1), i32(R), i32(cap),
            i32(cap // 128))  # fmt: skip


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_swiglu_experts_backward", mutates_args=())
def moe_swiglu_experts_backward(
    dy: torch.Tensor, xg: torch.Tensor, pre: torch.Tensor, act: torch.Tensor, out: torch.Tensor,
    weights: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor, pad_offsets: torch.Tensor,
    row_of_slot: torch.Tensor, slot_of_row: torch.Tensor, mtile_expert: torch.Tensor, row_align: int, need_x: bool,
    need_weights: bool, need_fc: bool, need_proj: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:  # fmt: skip
    """Returns (d_x, d_weights, d_w_fc, d_w_proj); a gradient that is not needed comes back empty."""
    T, top_k = weights.shape
    E = w_fc.size(0)
    maps = _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align)
    none = lambda: dy.new_empty(0)  # noqa: E731
    with torch.cuda.device(dy.device):
        d_out, d_w = K.combine_backward(dy.contiguous(), out, weights, maps, need_weights)
        d_w_proj = K.gemm_wgrad(d_out, act, E, pad_offsets) if need_proj else none()
        d_x, d_w_fc = none(), none()
        if need_x or need_fc:
            d_pre = K.gemm_dgrad_swiglu(d_out, w_proj, pre, mtile_expert, row_align)
            if need_fc:
                d_w_fc = K.gemm_wgrad(d_pre, xg, E, pad_offsets)
            if need_x:
                d_x = K.scatter_backward(K.gemm_dgrad(d_pre, w_fc, mtile_expert, row_align), maps, T)
    return d_x, (d_w if need_weights else none()), d_w_fc, d_w_proj


@moe_swiglu_experts_backward.register_fake
def _(dy, xg, pre, act, out, weights, w_fc, w_proj, pad_offsets, row_of_slot, slot_of_row, mtile_expert, row_align,
      need_x, need_weights, need_fc, need_proj):  # fmt: skip
    none = lambda: dy.new_empty(0)  # noqa: E731
    return (torch.empty_like(dy) if need_x else none(), torch.empty_like(weights) if need_weights else none(),
            torch.empty_like(w_fc) if need_fc else none(), torch.empty_like(w_proj) if need_proj else none())  # fmt: skip


def _experts_setup(ctx, inputs, output):
    _x, weights, _selected, _route_workspace, w_fc, w_proj, row_align = inputs
    _y, xg, pre, act, out, _count, pad_offsets, row_of_slot, slot_of_row, mtile_expert = output
    ctx.save_for_backward(xg, pre, act, out, weights, w_fc, w_proj, pad_offsets, row_of_slot, slot_of_row, mtile_expert)
    ctx.row_align = row_align


def _experts_backward(ctx, dy, *_unused):
    need_x, need_weights, _, _, need_fc, need_proj, _ = ctx.needs_input_grad
    d_x, d_w, d_w_fc, d_w_proj = moe_swiglu_experts_backward(
        dy, *ctx.saved_tensors, ctx.row_align, need_x, need_weights, need_fc, need_proj)  # fmt: skip
    return (d_x if need_x else None, d_w if need_weights else None, None, None, d_w_fc if need_fc else None,
            d_w_proj if need_proj else None, None)  # fmt: skip


torch.library.register_autograd(f"{LIBRARY_NAME}::moe_swiglu_experts", _experts_backward,
                                setup_context=_experts_setup)  # fmt: skip


# ---- general experts (any activation, optional bias): sort, scatter, expert linear, combine as separate ops ----
# Used by the traced layer when the activation is not swiglu_packed or the experts have a bias: the activation
# itself stays ordinary traced PyTorch code between two expert-linear ops.
@torch.library.custom_op(f"{LIBRARY_NAME}::moe_sort_maps", mutates_args=())
def moe_sort_maps(selected: torch.Tensor, route_workspace: torch.Tensor, num_experts: int,
                  row_align: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert)."""
    with torch.cuda.device(selected.device):
        m = K.moe_sort(selected, num_experts, row_align=row_align, routed_workspace=route_workspace)
    return m.expert_count, m.pad_offsets, m.row_of_slot, m.slot_of_row, m.mtile_expert


@moe_sort_maps.register_fake
def _(selected, route_workspace, num_experts, row_align):
    R = selected.numel()
    cap = K.rows_cap(R, num_experts, row_align)
    i32 = lambda *shape: selected.new_empty(shape, dtype=torch.int32)  # noqa: E731
    return (selected.new_empty((num_experts,), dtype=torch.uint32), i32(num_experts + 1), i32(R), i32(cap),
            i32(cap // 128))  # fmt: skip


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_scatter_rows", mutates_args=())
def moe_scatter_rows(x: torch.Tensor, pad_offsets: torch.Tensor, row_of_slot: torch.Tensor, slot_of_row: torch.Tensor,
                     mtile_expert: torch.Tensor, top_k: int, row_align: int) -> torch.Tensor:
    with torch.cuda.device(x.device):
        return K.scatter(x.contiguous(), _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align))


@moe_scatter_rows.register_fake
def _(x, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align):
    return x.new_empty(slot_of_row.size(0), x.size(1))


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_scatter_rows_backward", mutates_args=())
def moe_scatter_rows_backward(d_grouped: torch.Tensor, pad_offsets: torch.Tensor, row_of_slot: torch.Tensor,
                              slot_of_row: torch.Tensor, mtile_expert: torch.Tensor, top_k: int, row_align: int,
                              num_tokens: int) -> torch.Tensor:
    with torch.cuda.device(d_grouped.device):
        maps = _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align)
        return K.scatter_backward(d_grouped.contiguous(), maps, num_tokens)


@moe_scatter_rows_backward.register_fake
def _(d_grouped, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align, num_tokens):
    return d_grouped.new_empty(num_tokens, d_grouped.size(1))


def _scatter_setup(ctx, inputs, output):
    x, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align = inputs
    ctx.save_for_backward(pad_offsets, row_of_slot, slot_of_row, mtile_expert)
    ctx.top_k, ctx.row_align, ctx.num_tokens = top_k, row_align, x.size(0)


def _scatter_backward(ctx, d_grouped):
    d_x = moe_scatter_rows_backward(d_grouped, *ctx.saved_tensors, ctx.top_k, ctx.row_align, ctx.num_tokens)
    return d_x, None, None, None, None, None, None


torch.library.register_autograd(f"{LIBRARY_NAME}::moe_scatter_rows", _scatter_backward, setup_context=_scatter_setup)


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_expert_linear", mutates_args=())
def moe_expert_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, pad_offsets: torch.Tensor,
                      row_of_slot: torch.Tensor, slot_of_row: torch.Tensor, mtile_expert: torch.Tensor, top_k: int,
                      row_align: int) -> torch.Tensor:
    """y[p] = x[p] . weight[e(p)]^T (+ bias[e(p)] on token rows) over the grouped layout."""
    with torch.cuda.device(x.device):
        y = K.gemm_forward(x.contiguous(), weight.contiguous(), mtile_expert, row_align)
        if bias is not None:
            K.bias_add_(y, bias.contiguous(), _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align))
    return y


@moe_expert_linear.register_fake
def _(x, weight, bias, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align):
    return x.new_empty(x.size(0), weight.size(1))


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_expert_linear_backward", mutates_args=())
def moe_expert_linear_backward(d_y: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, pad_offsets: torch.Tensor,
                               row_of_slot: torch.Tensor, slot_of_row: torch.Tensor, mtile_expert: torch.Tensor,
                               top_k: int, row_align: int, need_x: bool, need_w: bool,
                               need_b: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (d_x, d_weight, d_bias); a gradient that is not needed comes back empty."""
    none = lambda: d_y.new_empty(0)  # noqa: E731
    with torch.cuda.device(d_y.device):
        d_y = d_y.contiguous()
        maps = _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align)
        d_x = K.gemm_dgrad(d_y, weight, mtile_expert, row_align) if need_x else none()
        d_w = K.gemm_wgrad(d_y, x, weight.size(0), pad_offsets) if need_w else none()
        d_b = K.bias_grad(d_y, maps) if need_b else none()
    return d_x, d_w, d_b


@moe_expert_linear_backward.register_fake
def _(d_y, x, weight, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align, need_x, need_w, need_b):
    none = lambda: d_y.new_empty(0)  # noqa: E731
    return (torch.empty_like(x) if need_x else none(), torch.empty_like(weight) if need_w else none(),
            d_y.new_empty(weight.size(0), weight.size(1)) if need_b else none())  # fmt: skip


def _linear_setup(ctx, inputs, output):
    x, weight, bias, pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align = inputs
    ctx.save_for_backward(x, weight, pad_offsets, row_of_slot, slot_of_row, mtile_expert)
    ctx.top_k, ctx.row_align, ctx.has_bias = top_k, row_align, bias is not None


def _linear_backward(ctx, d_y):
    x, weight, pad_offsets, row_of_slot, slot_of_row, mtile_expert = ctx.saved_tensors
    need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    need_b = ctx.has_bias and ctx.needs_input_grad[2]
    d_x, d_w, d_b = moe_expert_linear_backward(d_y, x, weight, pad_offsets, row_of_slot, slot_of_row, mtile_expert,
                                               ctx.top_k, ctx.row_align, need_x, need_w, need_b)  # fmt: skip
    return (d_x if need_x else None, d_w if need_w else None, d_b if need_b else None, None, None, None, None, None,
            None)  # fmt: skip


torch.library.register_autograd(f"{LIBRARY_NAME}::moe_expert_linear", _linear_backward, setup_context=_linear_setup)


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_combine_rows", mutates_args=())
def moe_combine_rows(expert_out: torch.Tensor, weights: torch.Tensor, pad_offsets: torch.Tensor,
                     row_of_slot: torch.Tensor, slot_of_row: torch.Tensor, mtile_expert: torch.Tensor,
                     row_align: int) -> torch.Tensor:
    T, top_k = weights.shape
    with torch.cuda.device(expert_out.device):
        maps = _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align)
        return K.combine(expert_out.contiguous(), weights.contiguous(), maps, T)


@moe_combine_rows.register_fake
def _(expert_out, weights, pad_offsets, row_of_slot, slot_of_row, mtile_expert, row_align):
    return expert_out.new_empty(weights.size(0), expert_out.size(1))


@torch.library.custom_op(f"{LIBRARY_NAME}::moe_combine_rows_backward", mutates_args=())
def moe_combine_rows_backward(dy: torch.Tensor, expert_out: torch.Tensor, weights: torch.Tensor,
                              pad_offsets: torch.Tensor, row_of_slot: torch.Tensor, slot_of_row: torch.Tensor,
                              mtile_expert: torch.Tensor, row_align: int,
                              need_weights: bool) -> tuple[torch.Tensor, torch.Tensor]:
    top_k = weights.size(1)
    with torch.cuda.device(dy.device):
        maps = _maps(pad_offsets, row_of_slot, slot_of_row, mtile_expert, top_k, row_align)
        d_out, d_w = K.combine_backward(dy.contiguous(), expert_out, weights, maps, need_weights)
    return d_out, (d_w if need_weights else dy.new_empty(0))


@moe_combine_rows_backward.register_fake
def _(dy, expert_out, weights, pad_offsets, row_of_slot, slot_of_row, mtile_expert, row_align, need_weights):
    return torch.empty_like(expert_out), (torch.empty_like(weights) if need_weights else dy.new_empty(0))


def _combine_setup(ctx, inputs, output):
    expert_out, weights, pad_offsets, row_of_slot, slot_of_row, mtile_expert, row_align = inputs
    ctx.save_for_backward(expert_out, weights, pad_offsets, row_of_slot, slot_of_row, mtile_expert)
    ctx.row_align = row_align


def _combine_backward(ctx, dy):
    need_w = ctx.needs_input_grad[1]
    d_out, d_w = moe_combine_rows_backward(dy, *ctx.saved_tensors, ctx.row_align, need_w)
    return d_out, (d_w if need_w else None), None, None, None, None, None


torch.library.register_autograd(f"{LIBRARY_NAME}::moe_combine_rows", _combine_backward, setup_context=_combine_setup)
