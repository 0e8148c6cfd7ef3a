"""Expert-parallel MoE on 2 GPUs against the single-GPU layer holding all experts, over both
transports: copy-engine pushes into peer-mapped arenas, and NCCL all-to-all.  Skipped on a box with
one GPU.  FMA_B200_TEST_PEER_FUSED=1 adds the variant whose GEMM epilogues store straight into the other
rank's arena; its store path is covered on one GPU by
test_gpu_gemm.py::test_bf16_peer_store_epilogue_into_local_buffers."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _worker(rank: int, world: int, port: int, result_dir: str):
    import torch.distributed as dist

    for p in (ROOT / "cute-kernels_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    import fma_b200
    from _util import randn

    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    try:
        dtype = torch.bfloat16
        T, H, E, k, I = 700, 256, 16, 4, 128
        full = fma_b200.MoE(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02)
        with torch.no_grad():
            full.gate.weight.copy_(randn((E, H), torch.float32, 1, 0.02))
            full.c_fc.weight.copy_(randn((E, 2 * I, H), torch.float32, 2, 0.02))
            full.c_proj.weight.copy_(randn((E, H, I), torch.float32, 3, 0.02))
        full = full.to(dev).to(dtype)
        xs = [randn((T + 64 * r, H), dtype, 10 + r).to(dev) for r in range(world)]  # ragged T per rank
        gs = [randn((T + 64 * r, H), dtype, 20 + r).to(dev) for r in range(world)]
        x_all = torch.cat(xs).requires_grad_(True)
        y_all, logits_all = full(x_all)
        y_all.backward(torch.cat(gs))
        lo = sum(t.size(0) for t in xs[:rank])
        hi = lo + xs[rank].size(0)

        shard = fma_b200.shard_expert_state_dict(full.state_dict(), rank, world)
        results = {}
        cases = ("peer", "nccl") + (("peer fused",) if os.environ.get("FMA_B200_TEST_PEER_FUSED") == "1" else ())
        for case in cases:
            # "peer fused": the down projection and the dgrad store their tiles straight into the senders' arenas
            transport = case.split()[0]
            ep = fma_b200.ExpertParallelMoE(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02, overlap_chunks=3,
                                            transport=transport, fuse_return=case.endswith("fused"))  # fmt: skip
            ep = ep.to(dev).to(dtype)
            ep.load_state_dict(shard, strict=True)
            for step in range(3):  # the arena is reused from the second step on
                for p in ep.parameters():
                    p.grad = None
                x = xs[rank].clone().requires_grad_(True)
                y, logits = ep(x)
                assert ep.last_transport == transport
                y.backward(gs[rank])
                torch.cuda.synchronize()
                assert torch.equal(logits, logits_all[lo:hi])
                e0, e1 = ep.local_expert_range()
                errs = {
                    "y": _rel(y, y_all[lo:hi]),
                    "dx": _rel(x.grad, x_all.grad[lo:hi]),
                    "d_w_fc": _rel(ep.c_fc.weight.grad, full.c_fc.weight.grad[e0:e1]),
                    "d_w_proj": _rel(ep.c_proj.weight.grad, full.c_proj.weight.grad[e0:e1]),
                }
                assert all(v <= 1e-2 for v in errs.values()), (case, step, errs)
                # y is a per-token computation: the expert-parallel result matches the local one bit for bit
                assert torch.equal(y, y_all[lo:hi])
            results[case] = (y, x.grad, ep.c_fc.weight.grad.clone(), ep.c_proj.weight.grad.clone())
            if case == "peer":
                # a second forward while the first one's backward is pending must not touch the arena
                x1 = xs[rank].clone().requires_grad_(True)
                y1, _ = ep(x1)
                x2 = xs[rank].clone().requires_grad_(True)
                y2, _ = ep(x2)
                assert ep.last_transport == "nccl"
                y2.backward(gs[rank])
                y1.backward(gs[rank])
                torch.cuda.synchronize()
                assert torch.equal(y1, y_all[lo:hi]) and torch.equal(y2, y_all[lo:hi])
                assert torch.equal(x1.grad, x2.grad)
                with torch.no_grad():
                    y3, _ = ep(xs[rank])
                assert ep.last_transport == "peer" and torch.equal(y3, y_all[lo:hi])
                ep.close_peer_transport()
            elif case == "peer fused":
                ep.close_peer_transport()
        # every variant computes each row with the same kernels: identical y and dx.  The weight gradients of the
        # variants whose receive layout keeps the sources apart (NCCL, fused return) reduce over ws segments per
        # expert and are identical to each other; the packed layout of the peer transport lines an expert's rows up
        # as the single-GPU layer does, so its weight gradients equal that layer's bit for bit.
        for case in cases:
            for a, b in zip(results[case][:2], results["nccl"][:2]):
                assert torch.equal(a, b), case
            if case != "peer":
                for a, b in zip(results[case][2:], results["nccl"][2:]):
                    assert torch.equal(a, b), case
        e0, e1 = ep.local_expert_range()
        assert torch.equal(results["peer"][2], full.c_fc.weight.grad[e0:e1])
        assert torch.equal(results["peer"][3], full.c_proj.weight.grad[e0:e1])
        from fma_b200 import _native

        assert _native.device_status() == 0
        Path(result_dir, f"ok{rank}").write_text(str(errs))
    finally:
        dist.destroy_process_group()


def _worker_general(rank: int, world: int, port: int, result_dir: str):
    """Experts with bias, and an activation other than SwiGLU: the expert-parallel layer runs them as separate
    differentiable steps; checked against the single-GPU layer holding all experts."""
    import torch.distributed as dist
    import torch.nn.functional as F

    for p in (ROOT / "cute-kernels_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    import fma_b200
    from _util import randn

    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    try:
        T, H, E, k, I = 500, 256, 8, 2, 128
        cases = {
            "gelu+bias bf16": (F.gelu, False, True, torch.bfloat16, 1e-2),
            "swiglu+bias f32": (fma_b200.swiglu_packed, True, True, torch.float32, 1e-5),
            "gelu f16": (F.gelu, False, False, torch.float16, 1e-2),
        }
        errs = {}
        for name, (act, glu, bias, dtype, tol) in cases.items():
            fc_out = 2 * I if glu else I
            full = fma_b200.MoE(E, k, H, I, act, glu, bias, 0.02)
            with torch.no_grad():
                full.gate.weight.copy_(randn((E, H), torch.float32, 1, 0.02))
                full.c_fc.weight.copy_(randn((E, fc_out, H), torch.float32, 2, 0.02))
                full.c_proj.weight.copy_(randn((E, H, I), torch.float32, 3, 0.02))
                if bias:
                    full.c_fc.bias.copy_(randn((E, fc_out), torch.float32, 4, 0.1))
                    full.c_proj.bias.copy_(randn((E, H), torch.float32, 5, 0.1))
            full = full.to(dev).to(dtype)
            xs = [randn((T + 32 * r, H), dtype, 10 + r).to(dev) for r in range(world)]
            gs = [randn((T + 32 * r, H), dtype, 20 + r).to(dev) for r in range(world)]
            x_all = torch.cat(xs).requires_grad_(True)
            y_all, logits_all = full(x_all)
            y_all.backward(torch.cat(gs))
            lo = sum(t.size(0) for t in xs[:rank])
            hi = lo + xs[rank].size(0)
            ep = fma_b200.ExpertParallelMoE(E, k, H, I, act, glu, bias, 0.02).to(dev).to(dtype)
            ep.load_state_dict(fma_b200.shard_expert_state_dict(full.state_dict(), rank, world), strict=True)
            x = xs[rank].clone().requires_grad_(True)
            y, logits = ep(x)
            assert ep.last_transport == "nccl"
            y.backward(gs[rank])
            torch.cuda.synchronize()
            assert torch.equal(logits, logits_all[lo:hi])
            assert torch.equal(y, y_all[lo:hi]), name  # per-token computation: same bits as the local layer
            e0, e1 = ep.local_expert_range()
            err = {
                "dx": _rel(x.grad, x_all.grad[lo:hi]),
                "d_w_fc": _rel(ep.c_fc.weight.grad, full.c_fc.weight.grad[e0:e1]),
                "d_w_proj": _rel(ep.c_proj.weight.grad, full.c_proj.weight.grad[e0:e1]),
            }
            if bias:
                err["d_b_fc"] = _rel(ep.c_fc.bias.grad, full.c_fc.bias.grad[e0:e1])
                err["d_b_proj"] = _rel(ep.c_proj.bias.grad, full.c_proj.bias.grad[e0:e1])
            assert all(v <= tol for v in err.values()), (name, err)
            errs[name] = err
        from fma_b200 import _native

        assert _native.device_status() == 0
        Path(result_dir, f"ok{rank}").write_text(str(errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_general_experts(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker_general, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_matches_single_gpu(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
