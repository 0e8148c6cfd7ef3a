"""Expert-parallel MoE: experts are sharded over the ranks of a process group, tokens stay
data-parallel, rows travel with all-to-all over NCCL (NVLink / NVSwitch).

The reference has no expert parallelism; this module keeps `MoE`'s interface and adds a process
group.  Rank r owns experts [r*E/ws, (r+1)*E/ws) (`c_fc.weight [E/ws, 2I, H]`,
`c_proj.weight [E/ws, H, I]`); the router `gate` is replicated.

The local experts are processed in `overlap_chunks` chunks: the all-to-all of chunk c+1 (and the
return exchange of chunk c-1) run on a high-priority side stream while the GEMMs of chunk c run, in the
forward and in the backward pass.  The GEMMs draw their tiles dynamically, so they keep going on the SMs
that the collective leaves free.

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

import os
from typing import Callable

import torch
import torch.distributed as dist

from .. import _native
from . import _kernels as K
from .moe import MoE, _Combine, _is_swiglu_packed, _Scatter

ROW_ALIGN = K.ROW_ALIGN
# transport="auto" uses the peer-memory transport up to this group size and NCCL all-to-all above it.
PEER_AUTO_MAX_RANKS = int(os.environ.get("FMA_B200_PEER_AUTO_MAX_RANKS", "8"))


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


def chunk_bounds(n_local_experts: int, n_chunks: int) -> list[int]:
    """Expert boundaries of the pipeline chunks.  The first dispatch and the last return exchange cannot
    hide behind any GEMM, so with 4 or more chunks the first and last chunk are made small (about 1/16
    of the experts each) and the middle ones share the rest evenly."""
    El = n_local_experts
    n_chunks = max(1, min(n_chunks, El))
    if n_chunks < 4 or El < 8:
        return [El * c // n_chunks for c in range(n_chunks + 1)]
    edge = max(1, El // 16)
    inner = n_chunks - 2
    rest = El - 2 * edge
    bounds = [0] + [edge + rest * c // inner for c in range(inner + 1)] + [El]
    return sorted(set(bounds))


class _ChunkPlan:
    """Host-side description of one forward's exchanges, split into chunks of local experts so that
    the all-to-all of one chunk runs while the GEMMs of another are busy.

    Built from the two count vectors after the single device-to-host copy of the layer."""

    def __init__(self, send_counts: list[int], recv_counts: list[list[int]], world_size: int, n_chunks: int):
        E = len(send_counts)
        El = E // world_size
        pad = lambda n: (n + ROW_ALIGN - 1) // ROW_ALIGN * ROW_ALIGN  # noqa: E731
        bounds = chunk_bounds(El, n_chunks)
        n_chunks = len(bounds) - 1
        self.world_size, self.n_chunks, self.bounds = world_size, n_chunks, bounds
        send_pad = [pad(n) for n in send_counts]
        offs = [0]
        for n in send_pad:
            offs.append(offs[-1] + n)
        self.total_send_rows = offs[-1]
        # rows of my grouped layout that go to rank r for chunk c: [start, start + rows)
        self.send_start = [[offs[r * El + bounds[c]] for r in range(world_size)] for c in range(n_chunks)]
        self.send_rows = [[offs[r * El + bounds[c + 1]] - offs[r * El + bounds[c]] for r in range(world_size)]
                          for c in range(n_chunks)]
        # rows that source s sends me for chunk c
        self.recv_rows = [[sum(pad(n) for n in recv_counts[s][bounds[c]:bounds[c + 1]]) for s in range(world_size)]
                          for c in range(n_chunks)]

    def experts(self, c: int) -> tuple[int, int]:
        return self.bounds[c], self.bounds[c + 1]


_comm_streams: dict[int, torch.cuda.Stream] = {}


def _comm_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _comm_streams:
        _comm_streams[idx] = torch.cuda.Stream(device=device, priority=-1)
    return _comm_streams[idx]


def _exchange_chunk(src: torch.Tensor, src_start: list[int], src_rows: list[int], dst: torch.Tensor,
                    dst_start: list[int], dst_rows: list[int], group) -> None:
    """One all-to-all: rows [src_start[r], +src_rows[r]) of `src` go to rank r; rows from rank s land at
    [dst_start[s], +dst_rows[s]) of `dst`."""
    ins = [src[a : a + n] for a, n in zip(src_start, src_rows)]
    outs = [dst[a : a + n] for a, n in zip(dst_start, dst_rows)]
    dist.all_to_all(outs, ins, group=group)


def _starts(rows: list[int]) -> list[int]:
    out, acc = [], 0
    for n in rows:
        out.append(acc)
        acc += n
    return out


class _EPFusedSwigluExperts(torch.autograd.Function):
    """Expert-parallel scatter -> dispatch -> grouped GEMMs -> combine, pipelined over chunks of local
    experts: exchanges run on a high-priority side stream and overlap the GEMMs of other chunks."""

    @staticmethod
    def forward(ctx, x, weights, w_fc, w_proj, maps: K.RowMaps, group, world_size: int, n_chunks: int):
        x = x.contiguous()
        weights = weights.contiguous()
        w_fc = w_fc.contiguous()
        w_proj = w_proj.contiguous()
        T, H = x.shape
        dev = x.device
        E_local = w_fc.size(0)
        main = torch.cuda.current_stream(dev)
        comm = _comm_stream(dev)

        recv_counts = exchange_counts(maps.expert_count, world_size, group)
        both = torch.cat([maps.expert_count.to(torch.int32), recv_counts.reshape(-1),
                          K.device_status_peek(dev)]).tolist()  # the one host sync; the status word rides along
        K.raise_for_device_status(both[-1:], "expert-parallel MoE")
        E = maps.num_experts
        plan = _ChunkPlan(both[:E], [both[E + s * E_local : E + (s + 1) * E_local] for s in range(world_size)],
                          world_size, n_chunks)
        C = plan.n_chunks

        xg = K.scatter(x, maps)
        ready = torch.cuda.Event()
        ready.record(main)

        recv, seg_offs, mtiles, pres, acts = [], [], [], [], []
        back = torch.empty(plan.total_send_rows, H, dtype=x.dtype, device=dev)
        back.record_stream(comm)
        xg.record_stream(comm)
        dispatched = [torch.cuda.Event() for _ in range(C)]
        combined = torch.cuda.Event()

        def dispatch(c: int) -> None:
            with torch.cuda.stream(comm):
                buf = torch.empty(sum(plan.recv_rows[c]), H, dtype=x.dtype, device=dev)
                buf.record_stream(main)
                _exchange_chunk(xg, plan.send_start[c], plan.send_rows[c], buf, _starts(plan.recv_rows[c]),
                                plan.recv_rows[c], group)
                dispatched[c].record(comm)
            recv.append(buf)

        with torch.cuda.stream(comm):
            comm.wait_event(ready)
        dispatch(0)
        if C > 1:
            dispatch(1)
        for c in range(C):
            e0, e1 = plan.experts(c)
            n_rows = recv[c].size(0)
            counts_c = recv_counts[:, e0:e1].contiguous()
            seg = torch.empty(world_size * (e1 - e0) + 1, dtype=torch.int32, device=dev)
            mt = torch.empty(max(n_rows // 128, 1), dtype=torch.int32, device=dev)
            K.call("fma_b200_moe_ep_recv_maps", K.ptr(counts_c), world_size, e1 - e0, ROW_ALIGN, n_rows, K.ptr(seg),
                   K.ptr(mt), K.stream_ptr(dev))  # fmt: skip
            main.wait_event(dispatched[c])
            pre, act = K.gemm_forward_swiglu(recv[c], w_fc[e0:e1], mt, keep_pre=True)
            out = K.gemm_forward(act, w_proj[e0:e1], mt)
            done = torch.cuda.Event()
            done.record(main)
            out.record_stream(comm)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                _exchange_chunk(out, _starts(plan.recv_rows[c]), plan.recv_rows[c], back, plan.send_start[c],
                                plan.send_rows[c], group)
                if c == C - 1:
                    combined.record(comm)
            if c + 2 < C:
                dispatch(c + 2)
            seg_offs.append(seg)
            mtiles.append(mt)
            pres.append(pre)
            acts.append(act)
        main.wait_event(combined)
        y = K.combine(back, weights, maps, T)

        ctx.save_for_backward(back, weights, w_fc, w_proj, *recv, *pres, *acts, *seg_offs, *mtiles)
        ctx.maps, ctx.group, ctx.world_size, ctx.T, ctx.plan = maps, group, world_size, T, plan
        return y

    @staticmethod
    def backward(ctx, dy):
        plan: _ChunkPlan = ctx.plan
        C = plan.n_chunks
        saved = ctx.saved_tensors
        back, weights, w_fc, w_proj = saved[:4]
        recv, pres, acts, seg_offs, mtiles = (saved[4 + i * C : 4 + (i + 1) * C] for i in range(5))
        maps, group, ws = ctx.maps, ctx.group, ctx.world_size
        dev = dy.device
        H = dy.size(1)
        main = torch.cuda.current_stream(dev)
        comm = _comm_stream(dev)
        need_x, need_w, need_fc, need_proj = ctx.needs_input_grad[:4]

        d_back, d_w = K.combine_backward(dy.contiguous(), back, weights, maps, need_w)
        ready = torch.cuda.Event()
        ready.record(main)
        d_back.record_stream(comm)
        d_w_fc = torch.empty_like(w_fc) if need_fc else None
        d_w_proj = torch.empty_like(w_proj) if need_proj else None
        d_xg = torch.empty(plan.total_send_rows, H, dtype=dy.dtype, device=dev) if need_x else None
        if d_xg is not None:
            d_xg.record_stream(comm)
        d_outs: list[torch.Tensor] = []
        dispatched = [torch.cuda.Event() for _ in range(C)]
        returned = torch.cuda.Event()

        def dispatch(c: int) -> None:
            with torch.cuda.stream(comm):
                buf = torch.empty(sum(plan.recv_rows[c]), H, dtype=dy.dtype, device=dev)
                buf.record_stream(main)
                _exchange_chunk(d_back, plan.send_start[c], plan.send_rows[c], buf, _starts(plan.recv_rows[c]),
                                plan.recv_rows[c], group)
                dispatched[c].record(comm)
            d_outs.append(buf)

        with torch.cuda.stream(comm):
            comm.wait_event(ready)
        dispatch(0)
        if C > 1:
            dispatch(1)
        for c in range(C):
            e0, e1 = plan.experts(c)
            main.wait_event(dispatched[c])
            d_out = d_outs[c]
            if need_proj:
                K.gemm_wgrad(d_out, acts[c], e1 - e0, seg_offs[c], n_seg=ws, out=d_w_proj[e0:e1])
            if need_x or need_fc:
                d_pre = K.gemm_dgrad_swiglu(d_out, w_proj[e0:e1], pres[c], mtiles[c])
                if need_fc:
                    K.gemm_wgrad(d_pre, recv[c], e1 - e0, seg_offs[c], n_seg=ws, out=d_w_fc[e0:e1])
                if need_x:
                    d_recv = K.gemm_dgrad(d_pre, w_fc[e0:e1], mtiles[c])
                    done = torch.cuda.Event()
                    done.record(main)
                    d_recv.record_stream(comm)
                    with torch.cuda.stream(comm):
                        comm.wait_event(done)
                        _exchange_chunk(d_recv, _starts(plan.recv_rows[c]), plan.recv_rows[c], d_xg,
                                        plan.send_start[c], plan.send_rows[c], group)
                        if c == C - 1:
                            returned.record(comm)
            if c + 2 < C:
                dispatch(c + 2)
        d_x = None
        if need_x:
            main.wait_event(returned)
            d_x = K.scatter_backward(d_xg, maps, ctx.T)
        return d_x, d_w, d_w_fc, d_w_proj, None, None, None, None


class _AllToAllRows(torch.autograd.Function):
    """Row exchange with a gradient: rows [0, sum(in_splits)) of the input go out, the result has `out_rows`
    rows of which the first sum(out_splits) are filled; the backward pass is the reverse exchange."""

    @staticmethod
    def forward(ctx, rows, in_splits, out_splits, out_rows, group):
        ctx.in_splits, ctx.out_splits, ctx.group, ctx.in_rows = in_splits, out_splits, group, rows.size(0)
        got = all_to_all_rows(rows.contiguous(), in_splits, out_splits, group)
        if got.size(0) == out_rows:
            return got
        out = torch.zeros(out_rows, rows.size(1), dtype=rows.dtype, device=rows.device)
        out[: got.size(0)] = got
        return out

    @staticmethod
    def backward(ctx, d_out):
        got = all_to_all_rows(d_out.contiguous(), ctx.out_splits, ctx.in_splits, ctx.group)
        if got.size(0) != ctx.in_rows:
            d_in = torch.zeros(ctx.in_rows, d_out.size(1), dtype=d_out.dtype, device=d_out.device)
            d_in[: got.size(0)] = got
            got = d_in
        return got, None, None, None, None


class _ExpertLinearReceived(torch.autograd.Function):
    """y[p] = x[p] . W[e(p)]^T (+ bias) over rows received from all ranks: the layout is
    [source rank][local expert] padded segments (`seg_offsets`), so an expert's rows lie in n_seg segments."""

    @staticmethod
    def forward(ctx, x, weight, bias, mtile_expert, seg_offsets, n_seg):
        x, weight = x.contiguous(), weight.contiguous()
        ctx.save_for_backward(x, weight, mtile_expert, seg_offsets)
        ctx.n_seg, ctx.has_bias = n_seg, bias is not None
        if x.size(0) == 0:  # this rank received nothing
            return x.new_empty(0, weight.size(1))
        y = K.gemm_forward(x, weight, mtile_expert, ROW_ALIGN)
        if bias is not None:
            # every row of a segment, padding included: padding rows of the received layout never reach a result
            # (the combine reads token rows only, and the gradients of padding rows are zero)
            all_rows = torch.zeros(x.size(0), dtype=torch.int32, device=x.device)
            K.call("fma_b200_moe_bias_add", K.ptr(y), K.ptr(bias.contiguous()), K.dtype_code(y.dtype), y.size(0), y.size(1),
                   K.ptr(mtile_expert), K.ptr(all_rows), K.stream_ptr(y.device))  # fmt: skip
        return y

    @staticmethod
    def backward(ctx, d_y):
        x, weight, mtile_expert, seg_offsets = ctx.saved_tensors
        d_y = d_y.contiguous()
        El, n_seg = weight.size(0), ctx.n_seg
        d_x = None
        if ctx.needs_input_grad[0]:
            d_x = K.gemm_dgrad(d_y, weight, mtile_expert, ROW_ALIGN) if d_y.size(0) > 0 else torch.empty_like(x)
        d_w = K.gemm_wgrad(d_y, x, El, seg_offsets, n_seg=n_seg) if ctx.needs_input_grad[1] else None
        d_b = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            acc = torch.zeros(El, d_y.size(1), dtype=torch.float32, device=d_y.device)
            if d_y.size(0) > 0:
                part = torch.empty(El, d_y.size(1), dtype=d_y.dtype, device=d_y.device)
                for s in range(n_seg):  # one column-sum pass per source rank's block of segments, in a fixed order
                    K.call("fma_b200_moe_bias_grad", K.ptr(d_y), K.dtype_code(d_y.dtype), El, d_y.size(1),
                           K.ptr(seg_offsets[s * El :]), K.ptr(part), K.stream_ptr(d_y.device))  # fmt: skip
                    acc += part.float()
            d_b = acc.to(d_y.dtype)
        return d_x, d_w, d_b, None, None, None


def peer_decision(table: list[list[int]], E: int) -> str:
    """What every rank does with the gathered rows [counts (E), rows_cap, arena in use, transport given up,
    status]: "unavailable" if any rank has given the peer transport up, "busy" if any rank's arena is still
    held by a pending backward (all ranks then take NCCL for this call), else "peer".  A pure function of
    the gathered table, so all ranks agree."""
    if any(row[E + 2] for row in table):
        return "unavailable"
    if any(row[E + 1] for row in table):
        return "busy"
    return "peer"


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
        overlap_chunks: int = 6,
        transport: str = "auto",
        capacity_factor: float = 1.5,
        fuse_return: bool = False,
    ) -> None:
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError(f"transport={transport!r}: expected 'auto', 'peer' or 'nccl'")
        self.process_group = process_group
        self.overlap_chunks = overlap_chunks
        self.transport = transport
        self.capacity_factor = capacity_factor
        # peer transport only: the down projection / dgrad store their tiles straight into the senders' arenas
        self.fuse_return = fuse_return
        self.last_transport = None  # "peer" or "nccl": what the most recent forward used
        self._arena = None
        self._sm_reserved = False
        self._peer_unavailable = None  # reason text once the peer transport has been given up
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
        maps = self._sort_selected(selected_experts)
        self.last_row_maps = maps
        fused = self.is_glu and _is_swiglu_packed(self.act) and self.c_fc.bias is None and self.c_proj.bias is None
        if not fused:
            self.last_transport = "nccl"
            return self._compute_experts_general(hidden_states, router_weights, maps)
        # "auto" takes the peer-memory transport only for the group size it has been validated on
        use_peer = self.transport == "peer" or (self.transport == "auto" and self.ep_size <= PEER_AUTO_MAX_RANKS)
        if use_peer:  # decided from the configuration alone: every rank enters the gather below or none does
            y = self._compute_experts_peer(hidden_states, router_weights, maps)
            if y is not None:
                self.last_transport = "peer"
                return y
        self.last_transport = "nccl"
        return _EPFusedSwigluExperts.apply(hidden_states, router_weights, self.c_fc.weight, self.c_proj.weight, maps,
                                           self.process_group, self.ep_size, self.overlap_chunks)  # fmt: skip

    def _compute_experts_general(self, hidden_states, router_weights, maps):
        """Any activation, optional bias, any dtype: scatter -> all-to-all -> expert linear -> activation ->
        expert linear -> all-to-all -> combine as separate differentiable steps over NCCL (no chunked overlap;
        the fused SwiGLU path above is the fast one)."""
        ws, group, dev = self.ep_size, self.process_group, hidden_states.device
        El = self.num_local_experts
        recv_counts = exchange_counts(maps.expert_count, ws, group)
        both = torch.cat([maps.expert_count.to(torch.int32), recv_counts.reshape(-1), K.device_status_peek(dev)]).tolist()
        K.raise_for_device_status(both[-1:], "expert-parallel MoE")
        E = self.num_experts
        pad = lambda n: (n + ROW_ALIGN - 1) // ROW_ALIGN * ROW_ALIGN  # noqa: E731
        send_rows = [sum(pad(n) for n in both[r * El : (r + 1) * El]) for r in range(ws)]
        recv_rows = [sum(pad(n) for n in both[E + s * El : E + (s + 1) * El]) for s in range(ws)]
        n_recv = sum(recv_rows)
        seg = torch.empty(ws * El + 1, dtype=torch.int32, device=dev)
        mt = torch.empty(max(n_recv // 128, 1), dtype=torch.int32, device=dev)
        K.call("fma_b200_moe_ep_recv_maps", K.ptr(recv_counts.contiguous()), ws, El, ROW_ALIGN, n_recv, K.ptr(seg),
               K.ptr(mt), K.stream_ptr(dev))  # fmt: skip
        xg = _Scatter.apply(hidden_states, maps)
        recv = _AllToAllRows.apply(xg, send_rows, recv_rows, n_recv, group)
        h = _ExpertLinearReceived.apply(recv, self.c_fc.weight, self.c_fc.bias, mt, seg, ws)
        h = self.act(h)
        out = _ExpertLinearReceived.apply(h, self.c_proj.weight, self.c_proj.bias, mt, seg, ws)
        back = _AllToAllRows.apply(out, recv_rows, send_rows, maps.rows_cap, group)
        return _Combine.apply(back, router_weights, maps, hidden_states.size(0))

    def _compute_experts_peer(self, hidden_states, router_weights, maps):
        """The layer over the peer-memory transport, or None when this call has to use NCCL: the arenas
        cannot be set up (transport="auto"), some rank's arena contents are still needed by a backward that
        has not run, or a rank would receive more rows than its arena holds.  Every rank takes the same
        decision: everything it depends on - the counts, the row capacity, and each rank's local state
        (arena in use, transport given up) - is in the row that the ranks gather.  The library's device
        status word rides along: if a kernel of the previous step recorded an error (a wait for a peer's
        rows that ran out, say), every rank raises instead of computing on rows that never arrived."""
        from . import moe_ep_peer as P

        dev = hidden_states.device
        E, ws = self.num_experts, self.ep_size
        arena = self._arena
        local_state = [maps.rows_cap, int(arena is not None and arena.busy), int(self._peer_unavailable is not None)]
        info = torch.cat([maps.expert_count.to(torch.int32), torch.tensor(local_state, dtype=torch.int32).to(dev, non_blocking=True),
                          K.device_status_peek(dev)])  # fmt: skip
        gathered = torch.empty(ws, E + 4, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(gathered, info, group=self.process_group)
        table = gathered.tolist()  # the one host synchronisation of the layer
        K.raise_for_device_status([row[E + 3] for row in table], "expert-parallel MoE (peer transport)")
        decision = peer_decision(table, E)
        if decision == "unavailable":
            self._peer_unavailable = self._peer_unavailable or "another rank has given up the peer transport"
            return None
        if decision == "busy":
            return None
        counts = [row[:E] for row in table]
        need = max(row[E] for row in table)
        H, dtype = hidden_states.size(1), hidden_states.dtype
        if arena is None or arena.send_cap < need or arena.hidden != H or arena.dtype != dtype:
            if arena is not None:
                arena.close()
                self._arena = None
            recv_cap = (int(self.capacity_factor * need) + 127) // 128 * 128
            try:
                arena = self._arena = P.PeerArena(self.process_group, dev, need, max(recv_cap, need), H, dtype)
            except P.PeerTransportUnavailable as e:
                if self.transport == "peer":
                    raise
                self._peer_unavailable = str(e)
                return None
        plan = P.PeerPlan(counts, self.ep_rank, self.overlap_chunks, expert_major=not self.fuse_return)
        if max(plan.total_recv_rows) > arena.recv_cap:  # the same plan on every rank
            return None
        if not self._sm_reserved:
            # The flag kernels of the side stream must find a free SM while a persistent grouped GEMM runs,
            # and a GEMM CTA fills its SM's shared memory: leave one CTA pair's worth of SMs out of the GEMM grids.
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            K.call("fma_b200_set_sm_limit", sms - 2)
            self._sm_reserved = True
        return P._EPPeerSwigluExperts.apply(hidden_states, router_weights, self.c_fc.weight, self.c_proj.weight, maps,
                                            arena, plan, gathered[:, :E].contiguous(), self.fuse_return)  # fmt: skip

    def close_peer_transport(self) -> None:
        """Collective: frees the peer-memory arena (the next forward would create a new one)."""
        if self._arena is not None:
            self._arena.close()
            self._arena = None


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
