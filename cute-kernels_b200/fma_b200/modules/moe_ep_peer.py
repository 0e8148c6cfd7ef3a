"""Peer-memory transport of the expert-parallel MoE (one node, NVLink / NVSwitch).

Instead of NCCL all-to-all kernels, which take SMs from the grouped GEMMs they overlap with, every
rank owns an arena that all ranks of the node map (CUDA IPC) and rows travel as copy-engine pushes
straight into the receiver's arena:

    sender, side stream:   copies (my padded segments -> the slot the receiver's layout reserves for
                           them), then one flag per receiver = sequence number of this layer call
    receiver, main stream: a small kernel waits (bounded) for the flags of the chunk, then the grouped
                           GEMMs read the rows in place: the arena region IS the GEMM operand.

Each rank knows every rank's per-expert row counts (one all-gather of E+1 integers per forward, which
is also the only host synchronisation and the cross-rank barrier that makes arena reuse safe), so
source and destination offsets of every block are computed on the host by `PeerPlan`, identically on
all ranks.

Arena regions (rows of H elements):
    recv     rows dispatched to my experts: expert after expert, inside an expert's block source after source
             with no padding between sources; the block as a whole is padded to the row alignment (rows of
             the padding are zeroed by the receiver).  With `expert_major=False` (what the GEMM epilogues that
             store into the senders' arenas need): [chunk][source rank][local expert] padded segments
    d_out    the same layout for the gradient rows dispatched in the backward pass
    back     expert outputs returned to me, in my own grouped layout (operand of the weighted combine)
    d_xg     gradient rows returned to me in the backward pass, same layout
"""

from __future__ import annotations

import ctypes
import os
import weakref

import torch
import torch.distributed as dist

from .. import _native
from . import _kernels as K
from .moe_ep import ROW_ALIGN, _comm_stream, chunk_bounds

MAX_CHUNKS = 16
MAX_RANKS = 64
REGIONS = ("recv", "d_out", "back", "d_xg")
FLAG_FWD_DISPATCH, FLAG_FWD_RETURN, FLAG_BWD_DISPATCH, FLAG_BWD_RETURN = range(4)
FLAG_BYTES = 4 * 4 * MAX_CHUNKS * MAX_RANKS
# Longest time a wait kernel polls for a peer's flag before it records the timeout status and returns.
WAIT_TIMEOUT_MS = int(os.environ.get("FMA_B200_PEER_TIMEOUT_MS", "2000"))


# Where the arena comes from: "ipc" = cudaMalloc + CUDA IPC through this library (every process then holds a
# context on every GPU whose arena it maps), "symm" = torch symmetric memory (driver virtual-memory API: peer
# memory is mapped into the process's own context).  Default: ipc for 2 ranks, symm above.
ARENA_ALLOCATOR = os.environ.get("FMA_B200_PEER_ALLOC", "auto")
# This transport uses plain peer loads and stores only.  Keep torch from binding the arena to an NVLink
# multicast object as well (it is never used here, and memory bound to one makes an abnormal exit of one
# rank a fault on the others); _allocate_symm refuses an arena that still came with one.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
_DEBUG = os.environ.get("FMA_B200_PEER_DEBUG", "0") == "1"
# Helper streams over which the copies of one push are spread (0 = all on the calling stream).
COPY_STREAMS = int(os.environ.get("FMA_B200_PEER_COPY_STREAMS", "8"))
_copy_stream_pool: dict[int, list] = {}


# "2": the dispatch of chunk c+2 is issued behind the return of chunk c on the one side stream (measured on 2, 4
# and 8 GPUs).  "all": every chunk's dispatch is issued at the start of a pass on a side stream of its own, so a
# dispatch never queues behind a return that waits for a GEMM (measured on 2 GPUs only: no difference there).
DISPATCH_AHEAD = os.environ.get("FMA_B200_PEER_DISPATCH_AHEAD", "2")
_dispatch_streams: dict[int, torch.cuda.Stream] = {}


def _dispatch_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _dispatch_streams:
        _dispatch_streams[idx] = torch.cuda.Stream(device=device, priority=-1)
    return _dispatch_streams[idx]


def _copy_streams(device: torch.device) -> list:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _copy_stream_pool:
        _copy_stream_pool[idx] = [torch.cuda.Stream(device=device, priority=-1) for _ in range(max(COPY_STREAMS, 0))]
    return _copy_stream_pool[idx]


def _debug(rank: int, text: str) -> None:
    """Progress lines of the collective set-up on stderr (FMA_B200_PEER_DEBUG=1): which phase a rank is in
    and how long the previous one took."""
    if _DEBUG:
        import sys
        import time

        print(f"[fma_b200 peer rank {rank} t={time.monotonic():.3f}] {text}", file=sys.stderr, flush=True)


class PeerTransportUnavailable(RuntimeError):
    """Raised on every rank of the group when the arenas could not be created or mapped."""


def _pad(n: int, align: int = ROW_ALIGN) -> int:
    return (n + align - 1) // align * align


def _prefix(values: list[int]) -> list[int]:
    out = [0]
    for v in values:
        out.append(out[-1] + v)
    return out


class PeerPlan:
    """Where every block of rows goes, from the matrix counts[s][e] = rows that rank s routes to
    (global) expert e.  Pure host arithmetic, the same on every rank.  Copies are (peer, dst_row, src_row, n_rows).

    expert_major=True (default): a receiver lays its rows out expert after expert; inside an expert's block the
    sources follow one another WITHOUT padding and the block is padded to `row_align` once.  One copy per
    (destination, expert).  The padding a receiver's GEMMs work through is then that of a single-GPU layer
    (half an alignment per expert) instead of half an alignment per expert AND source.

    expert_major=False: a block is the run of padded expert segments that one source sends to one destination
    for one chunk of the destination's local experts, shipped as it is ([chunk][source][expert], every segment
    padded): one copy per (destination, chunk), and every 128-row tile of the receive layout comes from one
    sender, which is what GEMM epilogues that store straight into the senders' arenas need."""

    def __init__(self, counts: list[list[int]], rank: int, n_chunks: int, row_align: int = ROW_ALIGN,
                 expert_major: bool = True):
        ws, E = len(counts), len(counts[0])
        if E % ws:
            raise ValueError(f"{E} experts over {ws} ranks")
        El = E // ws
        self.world_size, self.rank, self.num_local_experts = ws, rank, El
        self.expert_major = expert_major
        self.bounds = chunk_bounds(El, min(n_chunks, MAX_CHUNKS))
        C = self.n_chunks = len(self.bounds) - 1
        self.counts = counts
        # S[s][e]: first row of expert e in rank s's own grouped layout
        self.S = [_prefix([_pad(n, row_align) for n in row]) for row in counts]
        b = self.bounds
        self.total_send_rows = self.S[rank][E]
        if expert_major:
            # tot[r][j]: rows of r's local expert j over all sources; block[r][j]: first row of its block;
            # within[r][j][s]: offset of source s inside the block
            self.tot = [[sum(counts[s][r * El + j] for s in range(ws)) for j in range(El)] for r in range(ws)]
            self.block = [_prefix([_pad(n, row_align) for n in self.tot[r]]) for r in range(ws)]
            self.within = [[_prefix([counts[s][r * El + j] for s in range(ws)]) for j in range(El)] for r in range(ws)]
            self.recv_base = [[self.block[r][b[c]] for c in range(C + 1)] for r in range(ws)]
            self.total_recv_rows = [self.block[r][El] for r in range(ws)]
            return
        # rows[s][r][c]: size of the block s -> r, chunk c
        self.rows = [[[self.S[s][r * El + b[c + 1]] - self.S[s][r * El + b[c]] for c in range(C)] for r in range(ws)]
                     for s in range(ws)]  # fmt: skip
        # receive layout of rank r: chunk after chunk, inside a chunk source after source
        self.recv_base = [_prefix([sum(self.rows[s][r][c] for s in range(ws)) for c in range(C)]) for r in range(ws)]
        self.src_off = [[_prefix([self.rows[s][r][c] for s in range(ws)]) for c in range(C)] for r in range(ws)]
        self.total_recv_rows = [self.recv_base[r][C] for r in range(ws)]

    def experts(self, c: int) -> tuple[int, int]:
        return self.bounds[c], self.bounds[c + 1]

    def peer_order(self) -> list[int]:
        """Peers starting after this rank, this rank last: at any time the senders aim at different
        receivers."""
        return [(self.rank + 1 + i) % self.world_size for i in range(self.world_size)]

    def recv_chunk(self, c: int) -> tuple[int, int]:
        """(first row, rows) of chunk c in this rank's receive regions."""
        base = self.recv_base[self.rank]
        return base[c], base[c + 1] - base[c]

    def segments_per_expert(self) -> int:
        """Row segments an expert's rows form in the receive layout (the weight gradient reduces over them)."""
        return 1 if self.expert_major else self.world_size

    def padding_ranges(self, c: int) -> list[tuple[int, int]]:
        """expert_major: [first, end) rows of chunk c in this rank's receive regions that no sender writes (the
        padding at the end of every expert's block): the receiver zeroes them before its GEMMs read them."""
        if not self.expert_major:
            return []
        me, b = self.rank, self.bounds
        out = [(self.block[me][j] + self.tot[me][j], self.block[me][j + 1]) for j in range(b[c], b[c + 1])]
        return [(a, e) for a, e in out if e > a]

    def dispatch_copies(self, c: int) -> list[tuple[int, int, int, int]]:
        """My grouped layout -> the receive region of every rank."""
        me, El, b = self.rank, self.num_local_experts, self.bounds
        if self.expert_major:
            return [(r, self.block[r][j] + self.within[r][j][me], self.S[me][r * El + j], self.counts[me][r * El + j])
                    for r in self.peer_order() for j in range(b[c], b[c + 1]) if self.counts[me][r * El + j] > 0]  # fmt: skip
        return [(r, self.recv_base[r][c] + self.src_off[r][c][me], self.S[me][r * El + b[c]], self.rows[me][r][c])
                for r in self.peer_order()]  # fmt: skip

    def return_tiles(self, c: int) -> list[tuple[int, int]]:
        """For every 128-row tile of chunk c in this rank's receive layout: (rank it came from, first row of
        the tile in that rank's grouped layout) - where a fused GEMM epilogue has to store the tile."""
        if self.expert_major:
            raise ValueError("per-tile return addresses need expert_major=False: a tile of the packed layout mixes senders")
        me, El = self.rank, self.num_local_experts
        e0, e1 = self.experts(c)
        out = []
        for s in range(self.world_size):
            for e in range(me * El + e0, me * El + e1):
                first = self.S[s][e]
                out += [(s, first + 128 * j) for j in range((self.S[s][e + 1] - first) // 128)]
        return out

    def return_copies(self, c: int) -> list[tuple[int, int, int, int]]:
        """Rows of my chunk-local result (receive order) -> the grouped layout of the rank they came from."""
        me, El, b = self.rank, self.num_local_experts, self.bounds
        if self.expert_major:
            first = self.block[me][b[c]]
            return [(s, self.S[s][me * El + j], self.block[me][j] - first + self.within[me][j][s], self.counts[s][me * El + j])
                    for s in self.peer_order() for j in range(b[c], b[c + 1]) if self.counts[s][me * El + j] > 0]  # fmt: skip
        return [(s, self.S[s][me * El + b[c]], self.src_off[me][c][s], self.rows[s][me][c]) for s in self.peer_order()]


def _upload(array, device: torch.device) -> torch.Tensor:
    """Host array -> device tensor through pinned memory, asynchronously on the current stream."""
    return torch.from_numpy(array).pin_memory().to(device, non_blocking=True)


class _RawCudaMemory:
    """Exposes a raw device allocation through __cuda_array_interface__ so that torch can view it."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


class PeerArena:
    """One rank's arena plus the mappings of every other rank's arena.  Creation is collective."""

    def __init__(self, group, device: torch.device, send_cap: int, recv_cap: int, hidden: int, dtype: torch.dtype):
        self.group, self.device = group, device
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world_size > MAX_RANKS:
            raise RuntimeError(f"peer transport supports up to {MAX_RANKS} ranks")
        self.send_cap, self.recv_cap, self.hidden, self.dtype = send_cap, recv_cap, hidden, dtype
        self.row_bytes = hidden * torch.empty((), dtype=dtype).element_size()
        caps = {"recv": recv_cap, "d_out": recv_cap, "back": send_cap, "d_xg": send_cap}
        self.region_off, off = {}, FLAG_BYTES
        for name in REGIONS:
            self.region_off[name] = off
            off += _pad(caps[name] * self.row_bytes, 256)
        self.nbytes = off
        self.seq = 0
        self._lease = None

        self.local_ptr, self.peer_ptrs = 0, []
        self._symm = None  # (tensor, handle) when the arena comes from torch's symmetric memory
        allocator = ARENA_ALLOCATOR if ARENA_ALLOCATOR in ("ipc", "symm") else ("ipc" if self.world_size <= 2 else "symm")
        self.allocator = allocator
        if allocator == "symm":
            self._allocate_symm()
        else:
            self._allocate_ipc()
        raw = torch.as_tensor(_RawCudaMemory(self.local_ptr, self.nbytes), device=device)
        self.flags = raw[:FLAG_BYTES].view(torch.int32)
        self.regions = {
            name: raw[self.region_off[name] : self.region_off[name] + caps[name] * self.row_bytes].view(dtype).view(
                caps[name], hidden)
            for name in REGIONS
        }  # fmt: skip
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def _allocate_ipc(self) -> None:
        """cudaMalloc + CUDA IPC handles through the library's own entry points."""
        group, device = self.group, self.device
        local = ctypes.c_void_p()
        handle = (ctypes.c_uint8 * 64)()
        with torch.cuda.device(device):
            # every phase ends in a collective that all ranks reach, whether their part worked or not
            error = None
            _debug(self.rank, f"creating an arena of {self.nbytes >> 20} MiB")
            try:
                _native.call("fma_b200_peer_buffer_create", self.nbytes, ctypes.byref(local), handle)
                self.local_ptr = int(local.value)
            except RuntimeError as e:
                error = str(e)
            created = [None] * self.world_size
            dist.all_gather_object(created, (error, bytes(handle)), group=group)
            opened: list[int] = []
            _debug(self.rank, "arena created and handles gathered; mapping the peers' arenas")
            if error is None and all(err is None for err, _ in created):
                try:
                    for r, (_, h) in enumerate(created):
                        if r == self.rank:
                            opened.append(self.local_ptr)
                            continue
                        p = ctypes.c_void_p()
                        _native.call("fma_b200_peer_buffer_open", (ctypes.c_uint8 * 64).from_buffer_copy(h),
                                     ctypes.byref(p))  # fmt: skip
                        opened.append(int(p.value))
                except RuntimeError as e:
                    error = str(e)
            else:
                error = error or "another rank could not allocate its arena"
            errors = [None] * self.world_size
            dist.all_gather_object(errors, error, group=group)
            if any(e is not None for e in errors):
                for r, p in enumerate(opened):
                    if r != self.rank:
                        _native.lib().fma_b200_peer_buffer_close(ctypes.c_void_p(p))
                dist.barrier(group)
                if self.local_ptr:
                    _native.lib().fma_b200_peer_buffer_destroy(ctypes.c_void_p(self.local_ptr))
                    self.local_ptr = 0
                raise PeerTransportUnavailable("; ".join(f"rank {r}: {e}" for r, e in enumerate(errors) if e))
            self.peer_ptrs = opened
            _debug(self.rank, f"{len(opened) - 1} peer arenas mapped")

    def _allocate_symm(self) -> None:
        """Arena from torch.distributed._symmetric_memory (driver virtual-memory API, handles passed between
        the processes by torch): no CUDA IPC handles are involved.  Opt-in (FMA_B200_PEER_ALLOC=symm)."""
        import torch.distributed._symmetric_memory as symm_mem

        group = self.group if self.group is not None else dist.group.WORLD
        _debug(self.rank, f"allocating a symmetric arena of {self.nbytes >> 20} MiB")
        try:
            with torch.cuda.device(self.device):
                tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
                handle = symm_mem.rendezvous(tensor, group)
                tensor.zero_()
        except Exception as e:  # every rank fails or none: rendezvous is collective
            raise PeerTransportUnavailable(f"symmetric memory: {e}") from e
        if int(getattr(handle, "multicast_ptr", 0) or 0) != 0:
            # every rank sees the same: the binding is collective
            del handle, tensor
            raise PeerTransportUnavailable("symmetric memory came bound to an NVLink multicast object "
                                           "(TORCH_SYMM_MEM_DISABLE_MULTICAST had no effect)")
        self._symm = (tensor, handle)
        self.local_ptr = tensor.data_ptr()
        self.peer_ptrs = [int(p) for p in handle.buffer_ptrs]
        self.peer_ptrs[self.rank] = self.local_ptr
        _debug(self.rank, "symmetric arena mapped")

    # ---- lifetime ---------------------------------------------------------------------------
    def lease(self):
        """Token held by the autograd node of a forward whose regions the backward still needs."""

        class _Lease:
            pass

        token = _Lease()
        self._lease = weakref.ref(token)
        return token

    @property
    def busy(self) -> bool:
        return self._lease is not None and self._lease() is not None

    def close(self) -> None:
        """Collective: unmaps the peers' arenas and frees this rank's."""
        if self.local_ptr == 0:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        if self._symm is not None:
            self.flags, self.regions, self._symm = None, {}, None
            self.local_ptr, self.peer_ptrs = 0, []
            dist.barrier(self.group)
            return
        with torch.cuda.device(self.device):
            for r, p in enumerate(self.peer_ptrs):
                if r != self.rank:
                    _native.call("fma_b200_peer_buffer_close", ctypes.c_void_p(p))
            dist.barrier(self.group)
            self.flags, self.regions = None, {}
            _native.call("fma_b200_peer_buffer_destroy", ctypes.c_void_p(self.local_ptr))
        self.local_ptr, self.peer_ptrs = 0, []

    # ---- transport (all on the current stream) ------------------------------------------------
    @staticmethod
    def _flag_index(kind: int, chunk: int, src: int) -> int:
        return (kind * MAX_CHUNKS + chunk) * MAX_RANKS + src

    def _issue(self, copies: list[tuple[int, int, int, int]], base: int, off: int) -> None:
        n, rb = len(copies), self.row_bytes
        dst = (ctypes.c_uint64 * n)(*[self.peer_ptrs[r] + off + d * rb for r, d, _, _ in copies])
        srcs = (ctypes.c_uint64 * n)(*[base + s * rb for _, _, s, _ in copies])
        nbytes = (ctypes.c_int64 * n)(*[k * rb for _, _, _, k in copies])
        _native.call("fma_b200_peer_copy", n, dst, srcs, nbytes, _native.stream_ptr(self.device))

    def push(self, copies: list[tuple[int, int, int, int]], src: torch.Tensor, region: str) -> None:
        """copies = (peer, dst_row, src_row, n_rows): rows of `src` into `region` of each peer's arena.

        Copies issued on one stream run one after the other (measured on 2 GPUs: 33 MB peer copies at 70 us
        each, 480 GB/s, and the copies that stay on this GPU queue up behind them).  A list with more than a few
        copies is therefore dealt to COPY_STREAMS helper streams BY DESTINATION - all copies to one peer on one
        helper, the local ones on another - which start after the current stream's work and which the current
        stream waits for: copies to different destinations then run side by side on different copy engines and
        links.  (Copies to the same peer did not overlap one another when they were spread over streams.)"""
        copies = [c for c in copies if c[3] > 0]
        if not copies:
            return
        base, off = src.data_ptr(), self.region_off[region]
        helpers = _copy_streams(self.device) if len(copies) >= 8 else []
        if not helpers:
            self._issue(copies, base, off)
            return
        peers = list(dict.fromkeys(c[0] for c in copies))  # destinations in the order of the list
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for i, helper in enumerate(helpers):
            mine = set(peers[i :: len(helpers)])
            part = [c for c in copies if c[0] in mine]
            if not part:
                continue
            helper.wait_event(start)
            with torch.cuda.stream(helper):
                self._issue(part, base, off)
                done = torch.cuda.Event()
                done.record(helper)
            cur.wait_event(done)

    def zero_padding(self, region: str, base: int, seg_offsets: torch.Tensor, counts: torch.Tensor,
                     ranges: list[tuple[int, int]]) -> None:
        """Zeroes, on the current stream, the rows of this rank's own region that no sender writes: the padding at
        the end of every expert's block of the chunk that starts at row `base` (`seg_offsets` relative to it,
        `counts` rows per expert; `ranges` is the same thing as host numbers, for callers that model the arena)."""
        if not ranges:
            return
        view = self.regions[region][base:]
        K.call("fma_b200_moe_zero_padding", K.ptr(view), self.row_bytes, K.ptr(seg_offsets), K.ptr(counts),
               counts.numel(), K.stream_ptr(self.device))  # fmt: skip

    def return_tables(self, plan: PeerPlan) -> tuple[torch.Tensor, list[int]]:
        """Destination addresses for the GEMMs that store into the senders' arenas: an int64 device tensor
        [2, tiles] (row 0: into `back`, row 1: into `d_xg`) over all chunks, and the first tile of every chunk."""
        import numpy as np

        tiles, first = [], [0]
        for c in range(plan.n_chunks):
            tiles += plan.return_tiles(c)
            first.append(len(tiles))
        n = max(len(tiles), 1)
        table = np.zeros((2, n), dtype=np.int64)
        if tiles:
            base = np.array([self.peer_ptrs[s] for s, _ in tiles], dtype=np.int64)
            rows = np.array([row for _, row in tiles], dtype=np.int64)
            table[0, : len(tiles)] = base + self.region_off["back"] + rows * self.row_bytes
            table[1, : len(tiles)] = base + self.region_off["d_xg"] + rows * self.row_bytes
        return _upload(table, self.device), first

    def signal(self, kind: int, chunk: int, seq: int) -> None:
        n = self.world_size
        idx = 4 * self._flag_index(kind, chunk, self.rank)
        addrs = (ctypes.c_uint64 * n)(*[p + idx for p in self.peer_ptrs])
        _native.call("fma_b200_peer_signal", n, addrs, seq, _native.stream_ptr(self.device))

    def wait(self, kind: int, chunk: int, seq: int) -> None:
        first = self._flag_index(kind, chunk, 0)
        _native.call("fma_b200_peer_wait", ctypes.c_void_p(self.flags.data_ptr() + 4 * first), self.world_size, seq,
                     WAIT_TIMEOUT_MS, _native.stream_ptr(self.device))  # fmt: skip


class _EPPeerSwigluExperts(torch.autograd.Function):
    """scatter -> push to the expert ranks -> grouped GEMMs on the arena -> push back -> combine,
    pipelined over chunks of local experts; the backward mirrors it."""

    @staticmethod
    def forward(ctx, x, weights, w_fc, w_proj, maps: K.RowMaps, arena: PeerArena, plan: PeerPlan, counts_dev,
                fuse_return: bool = False):
        x, weights, w_fc, w_proj = x.contiguous(), weights.contiguous(), w_fc.contiguous(), w_proj.contiguous()
        T = x.size(0)
        dev = x.device
        me, ws, El, C = plan.rank, plan.world_size, plan.num_local_experts, plan.n_chunks
        main, comm = torch.cuda.current_stream(dev), _comm_stream(dev)
        arena.seq += 1
        seq = arena.seq

        # fuse_return: the down projection (and, in the backward pass, the dgrad) stores its tiles straight
        # into the arenas of the ranks the rows came from, so no result buffer and no return copies exist
        if fuse_return and plan.expert_major:
            raise ValueError("fuse_return needs a plan with expert_major=False")
        tables, first_tile = arena.return_tables(plan) if fuse_return else (None, None)
        n_seg = plan.segments_per_expert()
        if plan.expert_major:
            counts_local = counts_dev[:, me * El : (me + 1) * El].sum(0, dtype=torch.int32).reshape(1, El)
        else:
            counts_local = counts_dev[:, me * El : (me + 1) * El]
        xg = K.scatter(x, maps)
        ready = torch.cuda.Event()
        ready.record(main)
        ahead_all = DISPATCH_AHEAD == "all"
        disp = _dispatch_stream(dev) if ahead_all else comm
        xg.record_stream(disp)
        with torch.cuda.stream(disp):
            disp.wait_event(ready)

        def dispatch(c: int) -> None:
            with torch.cuda.stream(disp):
                arena.push(plan.dispatch_copies(c), xg, "recv")
                arena.signal(FLAG_FWD_DISPATCH, c, seq)

        for c in range(C if ahead_all else min(C, 2)):
            dispatch(c)
        recv, seg_offs, mtiles, pres, acts, chunk_counts = [], [], [], [], [], []
        for c in range(C):
            e0, e1 = plan.experts(c)
            base, n_rows = plan.recv_chunk(c)
            rows = arena.regions["recv"][base : base + n_rows]
            counts_c = counts_local[:, e0:e1].contiguous()
            seg = torch.empty(n_seg * (e1 - e0) + 1, dtype=torch.int32, device=dev)
            mt = torch.empty(max(n_rows // 128, 1), dtype=torch.int32, device=dev)
            K.call("fma_b200_moe_ep_recv_maps", K.ptr(counts_c), n_seg, e1 - e0, ROW_ALIGN, n_rows, K.ptr(seg), K.ptr(mt),
                   K.stream_ptr(dev))  # fmt: skip
            if plan.expert_major:
                arena.zero_padding("recv", base, seg, counts_c, plan.padding_ranges(c))
            arena.wait(FLAG_FWD_DISPATCH, c, seq)
            pre, act = K.gemm_forward_swiglu(rows, w_fc[e0:e1], mt, keep_pre=True)
            if fuse_return:
                K.gemm_forward_peer(act, w_proj[e0:e1], tables[0, first_tile[c] :], mt)
                arena.signal(FLAG_FWD_RETURN, c, seq)  # after the GEMM, in stream order
            else:
                out = K.gemm_forward(act, w_proj[e0:e1], mt)
                done = torch.cuda.Event()
                done.record(main)
                out.record_stream(comm)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    arena.push(plan.return_copies(c), out, "back")
                    arena.signal(FLAG_FWD_RETURN, c, seq)
            if not ahead_all and c + 2 < C:
                dispatch(c + 2)
            recv.append(rows)
            chunk_counts.append(counts_c)
            seg_offs.append(seg)
            mtiles.append(mt)
            pres.append(pre)
            acts.append(act)
        for c in range(C):
            arena.wait(FLAG_FWD_RETURN, c, seq)
        back = arena.regions["back"][: maps.rows_cap]
        y = K.combine(back, weights, maps, T)

        if any(ctx.needs_input_grad[:4]):
            ctx.lease = arena.lease()
        ctx.save_for_backward(back, weights, w_fc, w_proj, *recv, *pres, *acts, *seg_offs, *mtiles, *chunk_counts)
        ctx.maps, ctx.T, ctx.plan, ctx.arena, ctx.seq = maps, T, plan, arena, seq
        ctx.tables, ctx.first_tile = tables, first_tile
        return y

    @staticmethod
    def backward(ctx, dy):
        plan: PeerPlan = ctx.plan
        arena: PeerArena = ctx.arena
        C, ws, seq = plan.n_chunks, plan.world_size, ctx.seq
        saved = ctx.saved_tensors
        back, weights, w_fc, w_proj = saved[:4]
        recv, pres, acts, seg_offs, mtiles, chunk_counts = (saved[4 + i * C : 4 + (i + 1) * C] for i in range(6))
        maps = ctx.maps
        dev = dy.device
        main, comm = torch.cuda.current_stream(dev), _comm_stream(dev)
        need_x, need_w, need_fc, need_proj = ctx.needs_input_grad[:4]

        d_back, d_w = K.combine_backward(dy.contiguous(), back, weights, maps, need_w)
        ready = torch.cuda.Event()
        ready.record(main)
        ahead_all = DISPATCH_AHEAD == "all"
        disp = _dispatch_stream(dev) if ahead_all else comm
        d_back.record_stream(disp)
        with torch.cuda.stream(disp):
            disp.wait_event(ready)
        d_w_fc = torch.empty_like(w_fc) if need_fc else None
        d_w_proj = torch.empty_like(w_proj) if need_proj else None

        def dispatch(c: int) -> None:
            with torch.cuda.stream(disp):
                arena.push(plan.dispatch_copies(c), d_back, "d_out")
                arena.signal(FLAG_BWD_DISPATCH, c, seq)

        for c in range(C if ahead_all else min(C, 2)):
            dispatch(c)
        for c in range(C):
            e0, e1 = plan.experts(c)
            base, n_rows = plan.recv_chunk(c)
            if plan.expert_major:
                arena.zero_padding("d_out", base, seg_offs[c], chunk_counts[c], plan.padding_ranges(c))
            arena.wait(FLAG_BWD_DISPATCH, c, seq)
            d_out = arena.regions["d_out"][base : base + n_rows]
            n_seg = plan.segments_per_expert()
            if need_proj:
                K.gemm_wgrad(d_out, acts[c], e1 - e0, seg_offs[c], n_seg=n_seg, out=d_w_proj[e0:e1])
            d_pre = K.gemm_dgrad_swiglu(d_out, w_proj[e0:e1], pres[c], mtiles[c])
            if need_fc:
                K.gemm_wgrad(d_pre, recv[c], e1 - e0, seg_offs[c], n_seg=n_seg, out=d_w_fc[e0:e1])
            if ctx.tables is not None:
                K.gemm_dgrad_peer(d_pre, w_fc[e0:e1], ctx.tables[1, ctx.first_tile[c] :], mtiles[c])
                arena.signal(FLAG_BWD_RETURN, c, seq)
            else:
                d_recv = K.gemm_dgrad(d_pre, w_fc[e0:e1], mtiles[c])
                done = torch.cuda.Event()
                done.record(main)
                d_recv.record_stream(comm)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    arena.push(plan.return_copies(c), d_recv, "d_xg")
                    arena.signal(FLAG_BWD_RETURN, c, seq)
            if not ahead_all and c + 2 < C:
                dispatch(c + 2)
        # every rank waits for all returns even if it needs no input gradient: the peers' pushes into
        # this arena are then complete before the next layer call reuses it
        for c in range(C):
            arena.wait(FLAG_BWD_RETURN, c, seq)
        d_x = K.scatter_backward(arena.regions["d_xg"][: maps.rows_cap], maps, ctx.T) if need_x else None
        ctx.lease = None
        return d_x, d_w, d_w_fc, d_w_proj, None, None, None, None, None
