"""Expert-parallel MoE: experts are sharded over the ranks of a process group, tokens stay
data-parallel, rows travel with all-to-all over NCCL (NVLink / NVSwitch).

The reference has no expert parallelism; this module keeps `MoE`'s interface and adds a process
group.  Rank r owns experts [r*E/ws, (r+1)*E/ws) (`c_fc.weight [E/ws, 2I, H]`,
`c_proj.weight [E/ws, H, I]`); the router `gate` is replicated.

Per forward, with ws ranks and El = E/ws local experts:
  1. route + stable counting sort by GLOBAL expert id: rows for rank r are contiguous, and every
     expert segment is padded to 128 rows with zero rows (same layout as the 1-GPU path);
  2. counts all-to-all ([ws, El] int32) -> each rank knows the segments it receives; one small
     device-to-host copy gives the row split sizes NCCL needs;
  3. dispatch all-to-all of the padded segments: the receive buffer is [source rank][local expert]
     segments, each a multiple of 128 rows, so it is directly a grouped-GEMM operand (no regroup
     copy); weight gradients reduce over the ws segments of each expert inside the GEMM;
  4. grouped GEMMs (+SwiGLU epilogues) on the received rows;
  5. combine all-to-all back into the sender's padded layout, weighted combine there.
Backward runs the same two exchanges in reverse.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from ..kernel_backend import KernelBackend
from . import _kernels as K
from .moe import MoE, _is_swiglu_packed, _RouterTopK

ROW_ALIGN = K.ROW_ALIGN


def exchange_counts(expert_count: torch.Tensor, world_size: int, group) -> torch.Tensor:
    """All-to-all of per-expert row counts.  `expert_count` is [E] (int32/int64/uint32) on this rank;
    returns int32 [world_size, E_local]: rows that each source rank holds for this rank's experts."""
    E = expert_count.numel()
    send = expert_count.to(torch.int32).reshape(world_size, E // world_size).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def padded(n: torch.Tensor, align: int = ROW_ALIGN) -> torch.Tensor:
    return (n + (align - 1)) // align * align


def split_sizes(expert_count: torch.Tensor, recv_counts: torch.Tensor, world_size: int) -> tuple[list[int], list[int]]:
    """Rows (padded per expert) this rank sends to / receives from every rank.  Host lists; this is the
    one point where the expert-parallel path waits for the device."""
    E = expert_count.numel()
    send = padded(expert_count.to(torch.int64)).reshape(world_size, E // world_size).sum(1)
    recv = padded(recv_counts.to(torch.int64)).sum(1)
    both = torch.stack([send, recv]).tolist()
    return [int(v) for v in both[0]], [int(v) for v in both[1]]


def all_to_all_rows(rows: torch.Tensor, in_splits: list[int], out_splits: list[int], group) -> torch.Tensor:
    out = torch.empty(sum(out_splits), rows.size(1), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows[: sum(in_splits)], output_split_sizes=out_splits, input_split_sizes=in_splits,
                           group=group)  # fmt: skip
    return out


class _EPFusedSwigluExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, w_fc, w_proj, maps: K.RowMaps, group, world_size: int):
        x = x.contiguous()
        weights = weights.contiguous()
        w_fc = w_fc.contiguous()
        w_proj = w_proj.contiguous()
        T = x.size(0)
        E_local = w_fc.size(0)
        recv_counts = exchange_counts(maps.expert_count, world_size, group)
        send_rows, recv_rows = split_sizes(maps.expert_count, recv_counts, world_size)
        xg = K.scatter(x, maps)
        recv = all_to_all_rows(xg, send_rows, recv_rows, group)
        del xg
        n_rows = recv.size(0)
        dev = x.device
        seg_offsets = torch.empty(world_size * E_local + 1, dtype=torch.int32, device=dev)
        mtile_expert = torch.empty(max(n_rows // 128, 1), dtype=torch.int32, device=dev)
        K.call("fma_b200_moe_ep_recv_maps", K.ptr(recv_counts), world_size, E_local, ROW_ALIGN, n_rows,
               K.ptr(seg_offsets), K.ptr(mtile_expert), K.stream_ptr(dev))  # fmt: skip
        pre, act = K.gemm_forward_swiglu(recv, w_fc, mtile_expert, keep_pre=True)
        out = K.gemm_forward(act, w_proj, mtile_expert)
        back = all_to_all_rows(out, recv_rows, send_rows, group)
        del out
        # `back` has pad_offsets[E] rows; the combine kernels never index beyond that
        y = K.combine(back, weights, maps, T)
        ctx.save_for_backward(recv, pre, act, back, weights, w_fc, w_proj, seg_offsets, mtile_expert)
        ctx.maps, ctx.group, ctx.world_size, ctx.T = maps, group, world_size, T
        ctx.send_rows, ctx.recv_rows = send_rows, recv_rows
        return y

    @staticmethod
    def backward(ctx, dy):
        recv, pre, act, back, weights, w_fc, w_proj, seg_offsets, mtile_expert = ctx.saved_tensors
        maps, group, ws = ctx.maps, ctx.group, ctx.world_size
        E_local = w_fc.size(0)
        need_x, need_w, need_fc, need_proj = ctx.needs_input_grad[:4]
        d_back, d_w = K.combine_backward(dy.contiguous(), back, weights, maps, need_w)
        d_out = all_to_all_rows(d_back, ctx.send_rows, ctx.recv_rows, group)
        del d_back
        d_w_proj = K.gemm_wgrad(d_out, act, E_local, seg_offsets, n_seg=ws) if need_proj else None
        d_x = d_w_fc = None
        if need_x or need_fc:
            d_pre = K.gemm_dgrad_swiglu(d_out, w_proj, pre, mtile_expert)
            if need_fc:
                d_w_fc = K.gemm_wgrad(d_pre, recv, E_local, seg_offsets, n_seg=ws)
            if need_x:
                d_recv = K.gemm_dgrad(d_pre, w_fc, mtile_expert)
                d_xg = all_to_all_rows(d_recv, ctx.recv_rows, ctx.send_rows, group)
                d_x = K.scatter_backward(d_xg, maps, ctx.T)
        return d_x, d_w, d_w_fc, d_w_proj, None, None, None


class ExpertParallelMoE(MoE):
    """`MoE` whose experts are sharded over `process_group`.  `num_experts` is the GLOBAL expert count;
    this rank allocates num_experts / world_size of them.  With a group of size 1 it is `MoE`."""

    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: Callable,
        is_glu: bool,
        add_bias: bool,
        std: float,
        process_group=None,
    ) -> None:
        self.process_group = process_group
        self.ep_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.ep_rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        if num_experts % self.ep_size != 0:
            raise ValueError(f"num_experts={num_experts} is not divisible by the group size {self.ep_size}")
        local = num_experts // self.ep_size
        # build the local shard with the parent constructor, then restore the global routing width
        super().__init__(local, num_experts_per_tok, hidden_size, intermediate_size, activation_function, is_glu,
                         add_bias, std)  # fmt: skip
        self.num_local_experts = local
        self.num_experts = num_experts
        self.gate = torch.nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)

    def local_expert_range(self) -> tuple[int, int]:
        return self.ep_rank * self.num_local_experts, (self.ep_rank + 1) * self.num_local_experts

    def _compute_experts(self, hidden_states, router_weights, selected_experts):
        if self.ep_size == 1:
            return super()._compute_experts(hidden_states, router_weights, selected_experts)
        if not (self.is_glu and _is_swiglu_packed(self.act) and self.c_fc.bias is None):
            raise NotImplementedError("expert parallelism is implemented for SwiGLU experts without bias")
        with torch.no_grad():
            maps = K.moe_sort(selected_experts, self.num_experts)
        self.last_row_maps = maps
        return _EPFusedSwigluExperts.apply(hidden_states, router_weights, self.c_fc.weight, self.c_proj.weight, maps,
                                           self.process_group, self.ep_size)  # fmt: skip


def shard_expert_state_dict(full: dict, rank: int, world_size: int) -> dict:
    """Slices a full (all experts) MoE state dict into the shard of `rank`: expert tensors are cut along
    dim 0, the router weight is kept whole."""
    out = {}
    for key, value in full.items():
        if key.startswith(("c_fc.", "c_proj.")):
            n = value.size(0) // world_size
            out[key] = value[rank * n : (rank + 1) * n].clone()
        else:
            out[key] = value.clone()
    return out


def unshard_expert_state_dicts(shards: list[dict]) -> dict:
    """Inverse of shard_expert_state_dict: concatenates expert tensors of all ranks along dim 0."""
    out = {}
    for key, value in shards[0].items():
        if key.startswith(("c_fc.", "c_proj.")):
            out[key] = torch.cat([s[key] for s in shards], dim=0)
        else:
            out[key] = value.clone()
    return out
