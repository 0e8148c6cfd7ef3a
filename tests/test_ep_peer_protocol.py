"""The peer-memory transport's stream program, simulated on CPU for up to 8 ranks.

`_EPPeerSwigluExperts.forward/backward` (fma_b200.modules.moe_ep_peer) is run unchanged for every rank with
stand-ins for the CUDA pieces: streams become queues of deferred operations, events and flags become
readiness conditions, kernels become operations that CHECK the state they depend on instead of computing.
A scheduler then executes the queues of all ranks in random interleavings.  The test fails if
  * the program deadlocks (a wait whose flag nobody sets, an event nobody records),
  * a GEMM, combine or scatter-backward runs before every row it reads has arrived for THIS layer call
    (rows carry the sequence number of the push that wrote them, so a push of the next step that lands
    early is seen as well),
  * a push copies from a buffer whose producing kernel has not run.
Row placement itself is covered by test_ep_gloo.py::test_peer_plan_routes_every_block; the kernels by the
GPU tests.  The cross-rank barrier that the count all-gather provides at the start of every forward is
modelled as such: an operation on the main stream that completes when all ranks have reached it, and that
the host waits for before it issues the rest of the step.  (The program also passes with that barrier taken
out of the model: a rank can only push into a region after it has received what the previous reader of that
region produces, so the data dependencies alone order the reuse of the arenas.)"""

import random
import sys
from collections import deque
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "cute-kernels_b200"))

H = 4  # hidden size of the stand-in tensors (contents are never looked at)


class Sim:
    """Queues of deferred operations, one per (rank, stream)."""

    def __init__(self, world: int, seed: int):
        self.world = world
        self.rng = random.Random(seed)
        self.queues: dict[tuple[int, str], deque] = {}
        self.rank = 0  # rank whose host code is running
        self.current = {r: "main" for r in range(world)}
        self.executed = 0

    def enqueue(self, ready, run, what: str, stream: str | None = None):
        key = (self.rank, stream or self.current[self.rank])
        self.queues.setdefault(key, deque()).append((ready, run, what))

    def step(self) -> bool:
        """Runs one ready operation of a randomly chosen stream; False if none is ready."""
        keys = [k for k, q in self.queues.items() if q and q[0][0]()]
        if not keys:
            return False
        key = self.rng.choice(sorted(keys))
        _, run, _ = self.queues[key].popleft()
        run()
        self.executed += 1
        return True

    def run(self, until=None) -> None:
        while not (until and until()):
            if not self.step():
                pending = {k: q[0][2] for k, q in self.queues.items() if q}
                if until is None and not pending:
                    return
                raise AssertionError(f"deadlock: no operation is ready; heads of the queues: {pending}")

    def idle(self) -> bool:
        return not any(self.queues.values())


class FakeTensor(torch.Tensor):
    """CPU tensor that accepts record_stream and remembers whether its producer has run."""

    @staticmethod
    def make(rows: int, cols: int = H, ready: bool = False):
        t = torch.zeros(rows, cols).as_subclass(FakeTensor)
        t.state = {"ready": ready}
        return t

    def record_stream(self, stream):
        pass


def _state(t):
    """Producer state of a tensor or of the tensor a view was taken from."""
    while not hasattr(t, "state"):
        t = t._base
    return t.state


class FakeStream:
    def __init__(self, sim: Sim, rank: int, name: str):
        self.sim, self.rank, self.name = sim, rank, name

    def wait_event(self, event):
        self.sim.enqueue(lambda: event.done, lambda: None, f"wait_event on {self.name}", stream=self.name)


class FakeEvent:
    def __init__(self):
        self.done = False

    def record(self, stream: FakeStream):
        stream.sim.enqueue(lambda: True, lambda: setattr(self, "done", True), f"record on {stream.name}",
                           stream=stream.name)  # fmt: skip


class FakeArena:
    """Flags and per-row sequence numbers of one rank's arena; transport calls become queue operations."""

    def __init__(self, sim: Sim, rank: int, arenas: list, send_cap: int, recv_cap: int):
        self.sim, self.rank, self.arenas = sim, rank, arenas
        self.world_size = sim.world
        self.seq = 0
        caps = {"recv": recv_cap, "d_out": recv_cap, "back": send_cap, "d_xg": send_cap}
        self.regions = {name: FakeTensor.make(cap, ready=True) for name, cap in caps.items()}
        self.row_seq = {name: np.zeros(cap, dtype=np.int64) for name, cap in caps.items()}
        self.flags = np.zeros((4, 16, sim.world), dtype=np.int64)
        # made-up address space for the fused-return tables: rank r's arena starts at (r + 1) << 40
        self.device = torch.device("cpu")
        self.row_bytes = 2 * H
        self.peer_ptrs = [(r + 1) << 40 for r in range(sim.world)]
        self.region_off = {name: (i + 1) << 32 for i, name in enumerate(caps)}

    def return_tables(self, plan):
        from fma_b200.modules.moe_ep_peer import PeerArena

        return PeerArena.return_tables(self, plan)

    def zero_padding(self, region, base, seg_offsets, counts, ranges):
        seq = self.seq

        def run():
            for first, end in ranges:
                self.row_seq[region][first:end] = seq

        self.sim.enqueue(lambda: True, run, f"zero padding of {region}")

    def mark_tiles(self, table, n_tiles, seq):
        """What a GEMM with per-tile destinations does: 128 rows at every address of the table."""
        for addr in table[:n_tiles].tolist():
            peer, rest = (addr >> 40) - 1, addr & ((1 << 40) - 1)
            region = {off: name for name, off in self.region_off.items()}[rest >> 32 << 32]
            row = (rest & ((1 << 32) - 1)) // self.row_bytes
            self.arenas[peer].row_seq[region][row : row + 128] = seq

    def lease(self):
        return object()

    def region_of(self, view: torch.Tensor) -> tuple[str, int, int]:
        for name, t in self.regions.items():
            if view.untyped_storage().data_ptr() == t.untyped_storage().data_ptr():
                return name, view.storage_offset() // H, view.size(0)
        raise AssertionError("tensor is not a view of this arena")

    def push(self, copies, src, region):
        seq, me = self.seq, self.rank

        def run():
            assert _state(src)["ready"], f"rank {me}: push into {region} from a buffer whose kernel has not run"
            for peer, dst, s, n in copies:
                assert 0 <= s and s + n <= src.size(0)
                self.arenas[peer].row_seq[region][dst : dst + n] = seq

        self.sim.enqueue(lambda: True, run, f"push {region}")

    def signal(self, kind, chunk, seq):
        def run():
            for a in self.arenas:
                a.flags[kind, chunk, self.rank] = seq

        self.sim.enqueue(lambda: True, run, f"signal kind {kind} chunk {chunk}")

    def wait(self, kind, chunk, seq):
        self.sim.enqueue(lambda: bool((self.flags[kind, chunk] >= seq).all()), lambda: None,
                         f"wait kind {kind} chunk {chunk} seq {seq}")  # fmt: skip

    def check_rows(self, view, seq, what, n_rows=None):
        name, base, n = self.region_of(view)
        n = n if n_rows is None else n_rows
        got = self.row_seq[name][base : base + n]
        assert (got == seq).all(), (
            f"rank {self.rank}: {what} read rows of '{name}' that were not (only) written by call {seq}: "
            f"{sorted(set(got.tolist()))}")  # fmt: skip


def _install(monkeypatch, sim: Sim, arenas: list, plans: list):
    """Replaces the CUDA-facing names that moe_ep_peer uses by the simulation's."""
    from fma_b200.modules import moe_ep_peer as P

    streams = {(r, n): FakeStream(sim, r, n) for r in range(sim.world) for n in ("main", "comm", "disp")}

    class StreamContext:
        def __init__(self, stream):
            self.stream = stream

        def __enter__(self):
            self.prev = sim.current[sim.rank]
            sim.current[sim.rank] = self.stream.name

        def __exit__(self, *exc):
            sim.current[sim.rank] = self.prev

    monkeypatch.setattr(torch.cuda, "current_stream", lambda dev=None: streams[(sim.rank, sim.current[sim.rank])])
    monkeypatch.setattr(torch.cuda, "stream", StreamContext)
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    monkeypatch.setattr(P, "_comm_stream", lambda dev: streams[(sim.rank, "comm")])
    monkeypatch.setattr(P, "_dispatch_stream", lambda dev: streams[(sim.rank, "disp")])

    def kernel(out_rows, what, reads=(), arena_reads=()):
        """A stand-in kernel on the current stream: checks its inputs when it RUNS, then marks its output."""
        out = FakeTensor.make(out_rows)
        arena, seq = arenas[sim.rank], arenas[sim.rank].seq

        def run():
            for t in reads:
                assert _state(t)["ready"], f"rank {arena.rank}: {what} read a buffer whose kernel has not run"
            for view, n_rows in arena_reads:
                arena.check_rows(view, seq, what, n_rows)
            out.state["ready"] = True

        sim.enqueue(lambda: True, run, what)
        return out

    def in_arena(t):
        try:
            arenas[sim.rank].region_of(t)
            return True
        except AssertionError:
            return False

    def reads_of(*tensors):
        plain = [t for t in tensors if isinstance(t, FakeTensor) and not in_arena(t)]
        views = [(t, None) for t in tensors if isinstance(t, torch.Tensor) and t.numel() and in_arena(t)]
        return dict(reads=plain, arena_reads=views)

    K = P.K
    monkeypatch.setattr(K, "scatter", lambda x, maps: kernel(maps.rows_cap, "scatter"))
    monkeypatch.setattr(K, "call", lambda name, *a: kernel(1, name))
    monkeypatch.setattr(K, "ptr", lambda t: None)
    monkeypatch.setattr(K, "stream_ptr", lambda dev: None)

    def gemm_forward_swiglu(X, W, mt, keep_pre=True, row_align=256):
        pre = kernel(X.size(0), "up projection", **reads_of(X))
        return pre, pre

    monkeypatch.setattr(K, "gemm_forward_swiglu", gemm_forward_swiglu)
    monkeypatch.setattr(K, "gemm_forward", lambda X, W, mt, row_align=256: kernel(X.size(0), "down projection", **reads_of(X)))
    monkeypatch.setattr(K, "gemm_dgrad", lambda dY, W, mt, row_align=256: kernel(dY.size(0), "dgrad", **reads_of(dY)))
    monkeypatch.setattr(P, "_upload", lambda array, device: torch.from_numpy(array))

    def gemm_to_peers(what):
        def fn(X, W, table, mt, row_align=256):
            arena, seq, n_tiles = arenas[sim.rank], arenas[sim.rank].seq, X.size(0) // 128
            out = kernel(1, what, **reads_of(X))
            sim.enqueue(lambda: True, lambda: arena.mark_tiles(table, n_tiles, seq), what + " stores")
            return out

        return fn

    monkeypatch.setattr(K, "gemm_forward_peer", gemm_to_peers("down projection into the senders' arenas"))
    monkeypatch.setattr(K, "gemm_dgrad_peer", gemm_to_peers("dgrad into the senders' arenas"))
    monkeypatch.setattr(K, "gemm_dgrad_swiglu",
                        lambda d_out, W, pre, mt, row_align=256: kernel(d_out.size(0), "dgrad+swiglu", **reads_of(d_out, pre)))
    monkeypatch.setattr(K, "gemm_wgrad",
                        lambda dY, X, E, seg, n_seg=1, out=None: kernel(1, "wgrad", **reads_of(dY, X)))

    def own_layout_reads(view):
        """What the row movers read of a region in this rank's own grouped layout: with the packed receive layout
        only token rows travel back (the kernels never read the padding rows of an expert's segment)."""
        plan = plans[sim.rank]
        if not plan.expert_major:
            return [(view, plan.total_send_rows)]
        me = plan.rank
        return [(view[plan.S[me][e] : plan.S[me][e] + n], None) for e, n in enumerate(plan.counts[me]) if n > 0]

    def combine(back, weights, maps, T):
        return kernel(T, "combine", arena_reads=own_layout_reads(back))

    def combine_backward(dy, back, weights, maps, want):
        d_back = kernel(maps.rows_cap, "combine backward", arena_reads=own_layout_reads(back))
        return d_back, d_back

    def scatter_backward(d_xg, maps, T):
        return kernel(T, "scatter backward", arena_reads=own_layout_reads(d_xg))

    monkeypatch.setattr(K, "combine", combine)
    monkeypatch.setattr(K, "combine_backward", combine_backward)
    monkeypatch.setattr(K, "scatter_backward", scatter_backward)
    return P


class FakeCtx:
    needs_input_grad = (True, True, True, True, False, False, False, False)

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors


@pytest.mark.parametrize("ahead", ["2", "all"])
@pytest.mark.parametrize("fuse_return", [False, True])
@pytest.mark.parametrize("train", [True, False])
@pytest.mark.parametrize("world,experts,chunks,seed", [(2, 8, 3, 0), (4, 32, 6, 1), (8, 128, 6, 2), (8, 64, 8, 3), (3, 12, 1, 4)])
def test_peer_transport_program_is_live_and_ordered(monkeypatch, world, experts, chunks, seed, train, fuse_return, ahead):
    from fma_b200.modules import moe_ep_peer
    from fma_b200.modules.moe_ep_peer import PeerPlan

    monkeypatch.setattr(moe_ep_peer, "DISPATCH_AHEAD", ahead)

    rng = np.random.default_rng(seed)
    sim = Sim(world, seed)
    align = 256
    pad = lambda n: (n + align - 1) // align * align  # noqa: E731
    arenas: list = []
    plans: list = [None] * world
    P = _install(monkeypatch, sim, arenas, plans)
    n_steps = 3
    all_counts = [rng.integers(0, 3 * align, size=(world, experts)).tolist() for _ in range(n_steps)]
    for c in all_counts:  # an empty chunk on one rank, an expert nobody uses
        c[0][0] = 0
        for row in c:
            row[experts - 1] = 0
    send_cap = max(sum(pad(n) for n in row) for c in all_counts for row in c)
    recv_cap = max(max(PeerPlan(c, 0, chunks, align, expert_major=False).total_recv_rows) for c in all_counts)
    for r in range(world):
        arenas.append(FakeArena(sim, r, arenas, send_cap, recv_cap))
    barrier_count = [0] * (n_steps + 1)
    barrier_passed = [[False] * world for _ in range(n_steps + 1)]
    ctxs: list = [None] * world

    def maps_for(r, counts):
        rows = sum(pad(n) for n in counts[r])
        return SimpleNamespace(rows_cap=rows, num_experts=experts, expert_count=None)

    for step in range(n_steps):
        counts = all_counts[step]
        # the count all-gather: every rank's main stream reaches it, and the host waits for the result
        for r in range(world):
            sim.rank = r

            def arrive(step=step):
                barrier_count[step] += 1

            sim.enqueue(lambda: True, arrive, f"all-gather arrive {step}", stream="main")
            sim.enqueue(lambda step=step: barrier_count[step] == world,
                        lambda step=step, r=r: barrier_passed[step].__setitem__(r, True), f"all-gather {step}",
                        stream="main")  # fmt: skip
        sim.run(until=lambda step=step: all(barrier_passed[step]))
        # forward of every rank (host code only enqueues)
        for r in range(world):
            sim.rank = r
            plans[r] = PeerPlan(counts, r, chunks, align, expert_major=not fuse_return)
            ctxs[r] = FakeCtx()
            x = torch.zeros(5, H)
            P._EPPeerSwigluExperts.forward(ctxs[r], x, torch.zeros(5, 2), torch.zeros(experts // world, 2, H),
                                           torch.zeros(experts // world, H, 1), maps_for(r, counts), arenas[r], plans[r],
                                           torch.zeros(world, experts, dtype=torch.int32), fuse_return)  # fmt: skip
        if step % 2 == 0:  # sometimes the host is far ahead of the device, sometimes not
            sim.run(until=lambda: sim.rng.random() < 0.02 or sim.idle())
        if not train:  # forward-only calls back to back (evaluation): the arena is reused at once
            continue
        for r in range(world):
            sim.rank = r
            P._EPPeerSwigluExperts.backward(ctxs[r], torch.zeros(5, H))
        if step == 1:
            sim.run()
    sim.run()
    assert sim.idle() and sim.executed > 0
    for a in arenas:
        assert a.seq == n_steps
