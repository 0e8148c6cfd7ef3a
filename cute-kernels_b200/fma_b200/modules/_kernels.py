"""Thin Python calls into the C-ABI kernels of the MoE layer.  Every function allocates its
outputs with torch (the library itself allocates nothing) and launches on the current stream."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native
from .._native import call, dtype_code, ptr, stream_ptr

ROW_ALIGN = 256  # expert segments start on 256-row boundaries: one tile of a CTA pair (128 rows per CTA)


@dataclass
class RowMaps:
    """Row maps of the expert-contiguous layout for one routing decision."""

    expert_count: torch.Tensor  # uint32 [E]
    pad_offsets: torch.Tensor  # int32 [E+1]
    row_of_slot: torch.Tensor  # int32 [R]
    slot_of_row: torch.Tensor  # int32 [rows_cap]
    mtile_expert: torch.Tensor  # int32 [rows_cap/128]
    rows_cap: int
    num_experts: int
    top_k: int
    row_align: int = ROW_ALIGN
    sorted_expert_idxs: torch.Tensor | None = None  # int64 [R]
    sorted_scattered_idxs: torch.Tensor | None = None  # int64 [R]
    router_mean_prob: torch.Tensor | None = None  # float32 [E], when the router pass collected it


def device_status_peek(device: torch.device) -> torch.Tensor:
    """int32[1] device tensor holding a copy of the library's device status word (0 = no kernel reported an
    error), taken on the current stream without a host synchronisation and without clearing the word."""
    out = torch.empty(1, dtype=torch.int32, device=device)
    call("fma_b200_device_status_peek", ptr(out), stream_ptr(device))
    return out


STATUS_TEXT = {0x7001: "a grouped-GEMM barrier wait ran out", 0x7002: "a wait for a peer's rows ran out",
               0x7003: "the expert sort met an expert id outside [0, E)"}


def raise_for_device_status(codes, where: str) -> None:
    """`codes`: status words (one per rank, or one).  Clears the local word and raises if any is non-zero."""
    bad = {r: c for r, c in enumerate(codes) if c != 0}
    if not bad:
        return
    try:
        _native.device_status()  # clears the word so that the next step starts clean
    except RuntimeError:
        pass  # the error below is the one to report
    detail = ", ".join(f"rank {r}: {c:#x} ({STATUS_TEXT.get(c, 'unknown code')})" for r, c in bad.items())
    raise RuntimeError(f"{where}: a kernel recorded a device-side error in the previous step - {detail}")


def rows_cap(R: int, E: int, row_align: int = ROW_ALIGN) -> int:
    return int(_native.lib().fma_b200_moe_rows_cap(R, E, row_align))


def router_topk_softmax(logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    T, E = logits.shape
    logits = logits.contiguous()
    weights = torch.empty(T, k, dtype=logits.dtype, device=logits.device)
    selected = torch.empty(T, k, dtype=torch.int64, device=logits.device)
    call("fma_b200_router_topk_softmax", ptr(logits), dtype_code(logits.dtype), T, E, k, ptr(weights), ptr(selected),
         stream_ptr(logits.device))  # fmt: skip
    return weights, selected


def sort_workspace_bytes(R: int, E: int) -> int:
    return int(_native.lib().fma_b200_moe_sort_workspace_bytes(R, E))


def router_topk_softmax_routed(logits: torch.Tensor, k: int, want_probs: bool = False):
    """Top-k + softmax that also leaves the expert sort's first pass (and, with want_probs, the per-expert
    sums of the full softmax) in a workspace.  Returns (weights, selected, workspace): hand the workspace to
    moe_sort(..., routed_workspace=workspace) for the same `selected`."""
    T, E = logits.shape
    logits = logits.contiguous()
    weights = torch.empty(T, k, dtype=logits.dtype, device=logits.device)
    selected = torch.empty(T, k, dtype=torch.int64, device=logits.device)
    ws_bytes = sort_workspace_bytes(T * k, E)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=logits.device)
    call("fma_b200_router_topk_softmax_routed", ptr(logits), dtype_code(logits.dtype), T, E, k, ptr(weights),
         ptr(selected), int(want_probs), ptr(ws), ws_bytes, stream_ptr(logits.device))  # fmt: skip
    return weights, selected, ws


def router_mean_prob_backward(logits: torch.Tensor, d_mean_prob: torch.Tensor) -> torch.Tensor:
    """d_logits of mean_prob[e] = mean_t softmax(logits[t,:])[e] for an upstream gradient d_mean_prob [E]."""
    T, E = logits.shape
    logits = logits.contiguous()
    d_mean_prob = d_mean_prob.to(torch.float32).contiguous()
    d_logits = torch.empty_like(logits)
    call("fma_b200_router_mean_prob_backward", ptr(logits), ptr(d_mean_prob), dtype_code(logits.dtype), T, E,
         ptr(d_logits), stream_ptr(logits.device))  # fmt: skip
    return d_logits


def router_topk_softmax_backward(weights, d_weights, selected, E: int) -> torch.Tensor:
    T, k = weights.shape
    d_logits = torch.empty(T, E, dtype=weights.dtype, device=weights.device)
    call("fma_b200_router_topk_softmax_backward", ptr(weights), ptr(d_weights.contiguous()), ptr(selected),
         dtype_code(weights.dtype), T, E, k, ptr(d_logits), stream_ptr(weights.device))  # fmt: skip
    return d_logits


def moe_sort(selected: torch.Tensor, E: int, *, want_sorted: bool = False, row_align: int = ROW_ALIGN,
             routed_workspace: torch.Tensor | None = None, want_mean_prob: bool = False) -> RowMaps:
    """Stable counting sort of the selected expert ids [T,k] and the row maps of the grouped layout.
    `routed_workspace` is the workspace that router_topk_softmax_routed filled for these very ids (the
    histogram pass is then skipped); with want_mean_prob the router's mean probabilities are reduced too."""
    assert selected.dtype == torch.int64
    selected = selected.contiguous()
    dev = selected.device
    top_k = selected.size(-1) if selected.dim() > 1 else 1
    R = selected.numel()
    cap = rows_cap(R, E, row_align)
    expert_count = torch.empty(E, dtype=torch.uint32, device=dev)
    pad_offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    row_of_slot = torch.empty(R, dtype=torch.int32, device=dev)
    slot_of_row = torch.empty(cap, dtype=torch.int32, device=dev)
    mtile_expert = torch.empty(cap // 128, dtype=torch.int32, device=dev) if row_align % 128 == 0 else None
    sorted_e = torch.empty(R, dtype=torch.int64, device=dev) if want_sorted else None
    sorted_s = torch.empty(R, dtype=torch.int64, device=dev) if want_sorted else None
    ws_bytes = sort_workspace_bytes(R, E)
    mean_prob = None
    if routed_workspace is not None:
        assert selected.dim() == 2 and routed_workspace.numel() >= ws_bytes
        if want_mean_prob:
            mean_prob = torch.empty(E, dtype=torch.float32, device=dev)
        call("fma_b200_moe_sort_routed", ptr(selected), selected.size(0), top_k, E, row_align, cap, ptr(sorted_e),
             ptr(sorted_s), ptr(expert_count), ptr(pad_offsets), ptr(row_of_slot), ptr(slot_of_row), ptr(mtile_expert),
             ptr(mean_prob), ptr(routed_workspace), routed_workspace.numel(), stream_ptr(dev))  # fmt: skip
    else:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        call("fma_b200_moe_sort", ptr(selected), R, E, row_align, cap, ptr(sorted_e), ptr(sorted_s), ptr(expert_count),
             ptr(pad_offsets), ptr(row_of_slot), ptr(slot_of_row), ptr(mtile_expert), ptr(ws), ws_bytes,
             stream_ptr(dev))  # fmt: skip
    return RowMaps(expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert, cap, E, top_k, row_align, sorted_e,
                   sorted_s, mean_prob)


def scatter(x: torch.Tensor, maps: RowMaps) -> torch.Tensor:
    T, H = x.shape
    grouped = torch.empty(maps.rows_cap, H, dtype=x.dtype, device=x.device)
    call("fma_b200_moe_scatter", ptr(x), dtype_code(x.dtype), T, H, maps.top_k, ptr(maps.row_of_slot),
         ptr(maps.slot_of_row), ptr(maps.pad_offsets), maps.num_experts, maps.rows_cap, ptr(grouped),
         stream_ptr(x.device))  # fmt: skip
    return grouped


def scatter_backward(d_grouped: torch.Tensor, maps: RowMaps, T: int) -> torch.Tensor:
    H = d_grouped.size(1)
    dx = torch.empty(T, H, dtype=d_grouped.dtype, device=d_grouped.device)
    call("fma_b200_moe_scatter_backward", ptr(d_grouped), dtype_code(d_grouped.dtype), T, H, maps.top_k,
         ptr(maps.row_of_slot), ptr(dx), stream_ptr(dx.device))  # fmt: skip
    return dx


def combine(expert_out: torch.Tensor, weights: torch.Tensor, maps: RowMaps, T: int) -> torch.Tensor:
    H = expert_out.size(1)
    y = torch.empty(T, H, dtype=expert_out.dtype, device=expert_out.device)
    call("fma_b200_moe_combine", ptr(expert_out), ptr(weights), dtype_code(y.dtype), T, H, maps.top_k,
         ptr(maps.row_of_slot), ptr(y), stream_ptr(y.device))  # fmt: skip
    return y


def combine_backward(dy, expert_out, weights, maps: RowMaps, want_d_weights: bool = True):
    T, H = dy.shape
    d_out = torch.empty(maps.rows_cap, H, dtype=dy.dtype, device=dy.device)
    d_w = torch.empty_like(weights) if want_d_weights else None
    call("fma_b200_moe_combine_backward", ptr(dy), ptr(expert_out if want_d_weights else None), ptr(weights),
         dtype_code(dy.dtype), T, H, maps.top_k, ptr(maps.row_of_slot), ptr(maps.slot_of_row), ptr(maps.pad_offsets),
         maps.num_experts, maps.rows_cap, ptr(d_out), ptr(d_w), stream_ptr(dy.device))  # fmt: skip
    return d_out, d_w


def gemm_forward(X: torch.Tensor, W: torch.Tensor, mtile_expert: torch.Tensor, row_align: int = ROW_ALIGN) -> torch.Tensor:
    E, OUT, IN = W.shape
    rows = X.size(0)
    Y = torch.empty(rows, OUT, dtype=X.dtype, device=X.device)
    call("fma_b200_moe_gemm_forward", ptr(X), ptr(W), ptr(Y), dtype_code(X.dtype), rows, E, OUT, IN,
         ptr(mtile_expert), row_align, stream_ptr(X.device))  # fmt: skip
    return Y


def gemm_dgrad(dY: torch.Tensor, W: torch.Tensor, mtile_expert: torch.Tensor, row_align: int = ROW_ALIGN) -> torch.Tensor:
    E, OUT, IN = W.shape
    rows = dY.size(0)
    dX = torch.empty(rows, IN, dtype=dY.dtype, device=dY.device)
    call("fma_b200_moe_gemm_dgrad", ptr(dY), ptr(W), ptr(dX), dtype_code(dY.dtype), rows, E, OUT, IN,
         ptr(mtile_expert), row_align, stream_ptr(dY.device))  # fmt: skip
    return dX


def gemm_wgrad(dY: torch.Tensor, X: torch.Tensor, E: int, seg_offsets: torch.Tensor, n_seg: int = 1,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """dW[e] = dY_e^T . X_e; `out` (contiguous [E, OUT, IN]) receives the result when given."""
    rows, OUT = dY.shape
    IN = X.size(1)
    if rows == 0:  # no rows at all (an expert-parallel rank that received nothing)
        if out is not None:
            return out.zero_()
        return torch.zeros(E, OUT, IN, dtype=dY.dtype, device=dY.device)
    dW = out if out is not None else torch.empty(E, OUT, IN, dtype=dY.dtype, device=dY.device)
    assert dW.is_contiguous() and dW.shape == (E, OUT, IN)
    call("fma_b200_moe_gemm_wgrad", ptr(dY), ptr(X), ptr(dW), dtype_code(dY.dtype), rows, E, OUT, IN,
         ptr(seg_offsets), n_seg, stream_ptr(dY.device))  # fmt: skip
    return dW


def gemm_forward_swiglu(X: torch.Tensor, W: torch.Tensor, mtile_expert: torch.Tensor, keep_pre: bool = True,
                        row_align: int = ROW_ALIGN):
    """Up projection + SwiGLU.  bf16 / fp16: one fused tcgen05 kernel; f32: GEMM then the swiglu kernel."""
    E, twoI, IN = W.shape
    I = twoI // 2
    rows = X.size(0)
    dev = X.device
    if X.dtype in (torch.bfloat16, torch.float16):
        pre = torch.empty(rows, twoI, dtype=X.dtype, device=dev) if keep_pre else None
        act = torch.empty(rows, I, dtype=X.dtype, device=dev)
        call("fma_b200_moe_gemm_forward_swiglu", ptr(X), ptr(W), ptr(pre), ptr(act), dtype_code(X.dtype), rows, E, I,
             IN, ptr(mtile_expert), row_align, stream_ptr(dev))  # fmt: skip
        return pre, act
    pre = gemm_forward(X, W, mtile_expert, row_align)
    act = torch.empty(rows, I, dtype=X.dtype, device=dev)
    up, gate = pre[:, :I], pre[:, I:]
    call("fma_b200_swiglu_forward", ptr(gate), twoI, ptr(up), twoI, ptr(act), I, dtype_code(X.dtype), rows, I,
         stream_ptr(dev))  # fmt: skip
    return pre, act


def gemm_dgrad_swiglu(d_out: torch.Tensor, W: torch.Tensor, pre: torch.Tensor, mtile_expert: torch.Tensor,
                      row_align: int = ROW_ALIGN):
    """d_pre [rows, 2I] from d_out [rows, H]: dgrad of the down projection + SwiGLU backward."""
    E, OUT, I = W.shape
    rows = d_out.size(0)
    dev = d_out.device
    d_pre = torch.empty(rows, 2 * I, dtype=d_out.dtype, device=dev)
    if d_out.dtype in (torch.bfloat16, torch.float16):
        call("fma_b200_moe_gemm_dgrad_swiglu", ptr(d_out), ptr(W), ptr(pre), ptr(d_pre), dtype_code(d_out.dtype), rows,
             E, OUT, I, ptr(mtile_expert), row_align, stream_ptr(dev))  # fmt: skip
        return d_pre
    d_act = gemm_dgrad(d_out, W, mtile_expert, row_align)
    up, gate = pre[:, :I], pre[:, I:]
    d_up, d_gate = d_pre[:, :I], d_pre[:, I:]
    call("fma_b200_swiglu_backward", ptr(gate), 2 * I, ptr(up), 2 * I, ptr(d_act), I, ptr(d_gate), 2 * I, ptr(d_up),
         2 * I, dtype_code(d_out.dtype), rows, I, stream_ptr(dev))  # fmt: skip
    return d_pre


def bias_add_(grouped: torch.Tensor, bias: torch.Tensor, maps: RowMaps) -> torch.Tensor:
    """In place: grouped[p] += bias[expert(p)] on token rows (padding rows stay zero)."""
    rows, C = grouped.shape
    call("fma_b200_moe_bias_add", ptr(grouped), ptr(bias), dtype_code(grouped.dtype), rows, C, ptr(maps.mtile_expert),
         ptr(maps.slot_of_row), stream_ptr(grouped.device))  # fmt: skip
    return grouped


def bias_grad(d_grouped: torch.Tensor, maps: RowMaps) -> torch.Tensor:
    C = d_grouped.size(1)
    d_bias = torch.empty(maps.num_experts, C, dtype=d_grouped.dtype, device=d_grouped.device)
    call("fma_b200_moe_bias_grad", ptr(d_grouped), dtype_code(d_grouped.dtype), maps.num_experts, C,
         ptr(maps.pad_offsets), ptr(d_bias), stream_ptr(d_grouped.device))  # fmt: skip
    return d_bias


def gemm_forward_peer(X: torch.Tensor, W: torch.Tensor, dst_table: torch.Tensor, mtile_expert: torch.Tensor,
                      row_align: int = ROW_ALIGN) -> None:
    """gemm_forward whose 128-row output tiles are stored at the byte addresses in dst_table (int64, one per tile)."""
    E, OUT, IN = W.shape
    call("fma_b200_moe_gemm_forward_peer", ptr(X), ptr(W), ptr(dst_table), dtype_code(X.dtype), X.size(0), E, OUT, IN,
         ptr(mtile_expert), row_align, stream_ptr(X.device))  # fmt: skip


def gemm_dgrad_peer(dY: torch.Tensor, W: torch.Tensor, dst_table: torch.Tensor, mtile_expert: torch.Tensor,
                    row_align: int = ROW_ALIGN) -> None:
    """gemm_dgrad whose 128-row output tiles are stored at the byte addresses in dst_table (int64, one per tile)."""
    E, OUT, IN = W.shape
    call("fma_b200_moe_gemm_dgrad_peer", ptr(dY), ptr(W), ptr(dst_table), dtype_code(dY.dtype), dY.size(0), E, OUT, IN,
         ptr(mtile_expert), row_align, stream_ptr(dY.device))  # fmt: skip
