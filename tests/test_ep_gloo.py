"""Expert-parallel plumbing on CPU: two gloo ranks run the product's count exchange, split-size
computation and row all-to-all (fma_b200.modules.moe_ep) on padded grouped layouts, with the numpy
oracle standing in for the CUDA kernels, and must reproduce the single-process oracle output for
their own tokens."""

import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_dir: str):
    for p in (ROOT / "cute-kernels_b200", ROOT):
        sys.path.insert(0, str(p))
    from fma_b200.modules import moe_ep
    from oracle import moe_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        T, H, E, k, I = 150 + 37 * rank, 32, 8, 3, 16
        El = E // world
        rng = np.random.default_rng(5)  # weights: common to all ranks
        w_gate = rng.standard_normal((E, H), dtype=np.float32) * 0.5
        w_fc = rng.standard_normal((E, 2 * I, H), dtype=np.float32) * 0.1
        w_proj = rng.standard_normal((E, H, I), dtype=np.float32) * 0.1
        x = np.random.default_rng(100 + rank).standard_normal((T, H), dtype=np.float32)
        ref = O.moe_forward(x, w_gate, w_fc, w_proj, k, "f32")  # all experts, this rank's tokens

        align = moe_ep.ROW_ALIGN
        maps = O.row_maps(ref["selected"], E, align)
        total = int(maps["pad_offsets"][-1])
        xg = np.zeros((maps["rows_cap"], H), np.float32)
        xg[maps["row_of_slot"]] = np.repeat(x, k, axis=0)

        counts = torch.from_numpy(maps["expert_count"].astype(np.int64))
        recv_counts = moe_ep.exchange_counts(counts, world, None)
        assert recv_counts.shape == (world, El) and recv_counts.dtype == torch.int32
        # what every source really holds for my experts
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        for s in range(world):
            assert recv_counts[s].tolist() == gathered[s][rank * El : (rank + 1) * El].tolist()
        send_rows, recv_rows = moe_ep.split_sizes(counts, recv_counts, world)
        assert sum(send_rows) == total and all(r % align == 0 for r in send_rows + recv_rows)

        recv = moe_ep.all_to_all_rows(torch.from_numpy(xg), send_rows, recv_rows, None).numpy()
        # receive-side maps (what fma_b200_moe_ep_recv_maps computes on the GPU)
        seg = np.concatenate([[0], np.cumsum(-(-recv_counts.numpy().reshape(-1) // align) * align)])
        out = np.zeros((recv.shape[0], H), np.float32)
        for s in range(world):
            for e in range(El):
                a, n = seg[s * El + e], int(recv_counts[s, e])
                rows = recv[a : a + n]
                assert np.all(recv[a + n : seg[s * El + e + 1]] == 0)  # padding arrives as zeros
                ge = rank * El + e
                pre = rows @ w_fc[ge].T
                out[a : a + n] = O.swiglu_packed(pre, "f32") @ w_proj[ge].T
        back = moe_ep.all_to_all_rows(torch.from_numpy(out), recv_rows, send_rows, None).numpy()
        rows_of = maps["row_of_slot"].reshape(T, k)
        y = (back[rows_of] * ref["weights"][:, :, None]).sum(1)
        err = O.rel_l2(y, ref["y"])
        assert err < 1e-5, err
        Path(result_dir, f"ok{rank}").write_text(f"{err}")
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_two_gloo_ranks(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_and_unshard_state_dict_round_trip():
    sys.path.insert(0, str(ROOT / "cute-kernels_b200"))
    import fma_b200

    full = fma_b200.MoE(8, 2, 32, 16, fma_b200.swiglu_packed, True, False, 0.02).state_dict()
    shards = [fma_b200.shard_expert_state_dict(full, r, 4) for r in range(4)]
    assert shards[1]["c_fc.weight"].shape == (2, 32, 32) and shards[1]["gate.weight"].shape == (8, 32)
    assert torch.equal(shards[2]["c_proj.weight"], full["c_proj.weight"][4:6])
    back = fma_b200.unshard_expert_state_dicts(shards)
    assert list(back) == list(full)
    for key in full:
        assert torch.equal(back[key], full[key]), key
    # a shard loads strictly into an expert-parallel layer of the same local size (group size 1 here)
    local = fma_b200.MoE(2, 2, 32, 16, fma_b200.swiglu_packed, True, False, 0.02)
    sd = dict(shards[0])
    sd["gate.weight"] = sd["gate.weight"][:2]
    local.load_state_dict(sd, strict=True)


@pytest.mark.parametrize("expert_major", [True, False])
@pytest.mark.parametrize("world,E,chunks,align", [(2, 8, 1, 256), (3, 12, 4, 128), (4, 64, 6, 256), (8, 128, 6, 256)])
def test_peer_plan_routes_every_block(world, E, chunks, align, expert_major):
    """Host plan of the peer-memory transport: applying every rank's copy lists to emulated arenas (numpy) must
    build the receive layout on each rank - expert after expert with the sources packed inside a block and the
    block padded once (expert_major), or [chunk][source][expert] padded segments - and the return copies must
    rebuild every sender's own grouped layout."""
    sys.path.insert(0, str(ROOT / "cute-kernels_b200"))
    from fma_b200.modules.moe_ep_peer import PeerPlan

    rng = np.random.default_rng(world * 1000 + E)
    counts = rng.choice([0, 1, 7, align - 1, align, align + 1, 3 * align + 5], size=(world, E)).tolist()
    El = E // world
    plans = [PeerPlan(counts, r, chunks, align, expert_major=expert_major) for r in range(world)]
    pad = lambda n: (n + align - 1) // align * align  # noqa: E731

    # every rank's grouped layout: row label = s * 1e9 + e * 1e6 + i, padding rows -1
    def layout(s):
        rows = []
        for e in range(E):
            n = counts[s][e]
            rows += [s * 10**9 + e * 10**6 + i for i in range(n)] + [-1] * (pad(n) - n)
        return np.array(rows, dtype=np.int64)

    xg = [layout(s) for s in range(world)]
    for s in range(world):
        assert plans[s].total_send_rows == xg[s].size
    recv = [np.full(plans[0].total_recv_rows[r], -7, dtype=np.int64) for r in range(world)]
    for s in range(world):
        for c in range(plans[s].n_chunks):
            copies = plans[s].dispatch_copies(c)
            if not expert_major:
                assert sorted(r for r, *_ in copies) == list(range(world)) and copies[-1][0] == s
            for r, dst, src, n in copies:
                assert n > 0 or not expert_major
                assert np.all(recv[r][dst : dst + n] == -7)  # no two blocks overlap
                recv[r][dst : dst + n] = xg[s][src : src + n]
    for r in range(world):
        for c in range(plans[r].n_chunks):  # the receiver zeroes what no sender writes
            for first, end in plans[r].padding_ranges(c):
                base, n_rows = plans[r].recv_chunk(c)
                assert base <= first < end <= base + n_rows
                assert np.all(recv[r][first:end] == -7)
                recv[r][first:end] = -1
        assert not np.any(recv[r] == -7)  # every row of the receive layout was written
        for c in range(plans[r].n_chunks):
            e0, e1 = plans[r].experts(c)
            base, n_rows = plans[r].recv_chunk(c)
            want = []
            if expert_major:
                for e in range(r * El + e0, r * El + e1):
                    block = [xg[s][sum(pad(v) for v in counts[s][:e]) :][: counts[s][e]] for s in range(world)]
                    n = sum(b.size for b in block)
                    want += block + [np.full(pad(n) - n, -1, dtype=np.int64)]
            else:
                for s in range(world):
                    for e in range(r * El + e0, r * El + e1):
                        first = sum(pad(v) for v in counts[s][:e])
                        want.append(xg[s][first : first + pad(counts[s][e])])
            want = np.concatenate(want) if want else np.zeros(0, np.int64)
            assert n_rows == want.size and n_rows % 128 == 0
            np.testing.assert_array_equal(recv[r][base : base + n_rows], want)
    back = [np.full(xg[s].size, -7 if not expert_major else -1, dtype=np.int64) for s in range(world)]
    for r in range(world):
        for c in range(plans[r].n_chunks):
            base, n_rows = plans[r].recv_chunk(c)
            out = recv[r][base : base + n_rows]  # identity "experts"
            for s, dst, src, n in plans[r].return_copies(c):
                back[s][dst : dst + n] = out[src : src + n]
    for s in range(world):
        # expert_major returns the token rows only: the padding rows of a sender's layout are never read
        np.testing.assert_array_equal(back[s], xg[s])
    if expert_major:  # the packed layout is never larger than the per-source padded one
        other = PeerPlan(counts, 0, chunks, align, expert_major=False)
        assert all(a <= b for a, b in zip(plans[0].total_recv_rows, other.total_recv_rows))


def test_chunk_bounds_cover_all_experts():
    """Pipeline chunks: strictly increasing bounds from 0 to the expert count, never more chunks than
    experts, small first and last chunk once there are at least 4 chunks and 8 experts."""
    sys.path.insert(0, str(ROOT / "cute-kernels_b200"))
    from fma_b200.modules.moe_ep import chunk_bounds

    for experts in (1, 2, 3, 7, 8, 16, 32, 64, 128):
        for chunks in (1, 2, 3, 4, 6, 8, 16, 200):
            b = chunk_bounds(experts, chunks)
            assert b[0] == 0 and b[-1] == experts and all(x < y for x, y in zip(b, b[1:]))
            assert len(b) - 1 <= min(chunks, experts)
            if chunks >= 4 and experts >= 8:
                sizes = [y - x for x, y in zip(b, b[1:])]
                assert sizes[0] == sizes[-1] == max(1, experts // 16)
                assert max(sizes[1:-1]) - min(sizes[1:-1]) <= 1


def test_transport_decision_is_a_function_of_the_gathered_table_only():
    """Ranks whose LOCAL state differs (one arena still held by a pending backward, one rank that has given
    the peer transport up) must still take the same branch: the decision reads nothing but the table that
    all ranks gathered, and "given up" wins over "busy" wins over "peer"."""
    from fma_b200.modules import _kernels as K
    from fma_b200.modules.moe_ep import peer_decision

    E = 4
    row = lambda busy, gone, status=0: [10, 20, 30, 40, 1024, busy, gone, status]  # noqa: E731
    assert peer_decision([row(0, 0), row(0, 0)], E) == "peer"
    assert peer_decision([row(0, 0), row(1, 0)], E) == "busy"  # only rank 1 is busy: both take NCCL
    assert peer_decision([row(1, 0), row(0, 0), row(0, 0)], E) == "busy"
    assert peer_decision([row(0, 0), row(0, 1)], E) == "unavailable"
    assert peer_decision([row(1, 0), row(0, 1)], E) == "unavailable"
    # the status word of the previous step: any non-zero code makes every rank raise, naming rank and code
    K.raise_for_device_status([0, 0], "test")
    with pytest.raises(RuntimeError, match=r"rank 1: 0x7002"):
        K.raise_for_device_status([0, 0x7002], "test")
