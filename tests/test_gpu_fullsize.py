"""The layer at the full sizes of the benchmark configurations (Mixtral-shaped, fine-grained, and the
per-GPU shape of the expert-parallel one, which is what the benchmark times), where the CPU oracle
cannot evaluate the whole layer in seconds.  Checked through size-independent properties, plus the
oracle on samples:
  * determinism: two runs give identical bits (no floating-point atomics anywhere);
  * token-permutation equivariance: y and dx follow a permutation of the tokens bit for bit, weight
    gradients keep their value up to summation order;
  * exact scaling: a backward pass with 2*dy gives exactly 2x every gradient (powers of two commute
    with every rounding step);
  * conservation: expert counts sum to T*k, every token slot owns exactly one grouped row;
  * sampled parity, forward and backward: for a sample of tokens the oracle (their experts, same logits)
    reproduces y and dx (a token's output and input gradient depend on that token alone); for the
    most loaded, a median and the least loaded expert the oracle, run on all rows of that expert,
    reproduces its two weight gradients.  rel-L2 <= 1e-2 (bf16).
"""

import numpy as np
import pytest
import torch

from _util import DEV, check_device_status, rel_l2, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

CONFIGS = {
    "mixtral_shaped": dict(T=16384, H=4096, E=8, k=2, I=14336, zipf=False, sample=48),
    "fine_grained_zipf": dict(T=32768, H=2048, E=128, k=8, I=768, zipf=True, sample=48),
    # one GPU's share of the expert-parallel configuration with all 128 experts local: the benchmarked shape
    "expert_parallel_per_gpu": dict(T=65536, H=4096, E=128, k=8, I=1536, zipf=False, sample=8),
}


def _layer(cfg):
    import fma_b200

    E, k, H, I = cfg["E"], cfg["k"], cfg["H"], cfg["I"]
    with torch.device("meta"):
        moe = fma_b200.MoE(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02)
    moe = moe.to_empty(device=DEV).to(torch.bfloat16)
    g = torch.Generator(device=DEV).manual_seed(1)
    with torch.no_grad():
        for w in (moe.gate.weight, moe.c_fc.weight, moe.c_proj.weight):
            for e in range(w.size(0)):  # expert by expert: bounded temporary
                w[e].copy_(torch.randn(w.shape[1:], generator=g, device=DEV) * 0.02)
        for m in (moe.c_fc, moe.c_proj):
            m.N_array.fill_(m.out_features)
            m.K_array.fill_(m.in_features)
        if cfg["zipf"]:
            gate = torch.nn.Linear(H, E, bias=True, device=DEV, dtype=torch.bfloat16)
            p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64)
            perm = torch.randperm(E, generator=torch.Generator().manual_seed(3))
            gate.weight.copy_(moe.gate.weight)
            gate.bias.copy_(torch.log(p / p.sum())[perm].to(torch.bfloat16))
            moe.gate = gate
    return moe


def _step(moe, x, dy):
    for p in moe.parameters():
        p.grad = None
    x = x.detach().clone().requires_grad_(True)
    y, logits = moe(x)
    y.backward(dy)
    return y.detach(), logits.detach(), x.grad, moe.c_fc.weight.grad, moe.c_proj.weight.grad


@pytest.mark.parametrize("name", list(CONFIGS))
def test_full_size_properties(name):
    cfg = CONFIGS[name]
    T, H, E, k = cfg["T"], cfg["H"], cfg["E"], cfg["k"]
    moe = _layer(cfg)
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    dy = torch.randn(T, H, generator=g, device=DEV).bfloat16()

    y, logits, dx, dfc, dproj = _step(moe, x, dy)
    check_device_status()
    maps = moe.last_row_maps
    cnt = to_np(maps.expert_count)
    assert cnt.sum() == T * k
    rows = to_np(maps.row_of_slot)
    assert len(np.unique(rows)) == T * k  # one grouped row per token slot
    slots = to_np(maps.slot_of_row)
    assert np.array_equal(slots[rows], np.arange(T * k))
    assert (slots >= 0).sum() == T * k
    if cfg["zipf"]:
        assert cnt.max() > 20 * max(1, np.median(cnt))  # the load really is skewed
    for t in (y, dx, dfc, dproj):
        assert torch.isfinite(t).all()

    # determinism
    y2, _, dx2, dfc2, dproj2 = _step(moe, x, dy)
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(dfc, dfc2) and torch.equal(dproj, dproj2)

    # exact scaling of the backward pass
    _, _, dx3, dfc3, dproj3 = _step(moe, x, dy * 2)
    assert torch.equal(dx3, dx * 2) and torch.equal(dfc3, dfc * 2) and torch.equal(dproj3, dproj * 2)
    del dx3, dfc3, dproj3, y2, dx2, dfc2, dproj2

    # token-permutation equivariance
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(5)).to(DEV)
    yp, lp, dxp, dfcp, dprojp = _step(moe, x[perm], dy[perm])
    assert torch.equal(lp, logits[perm])
    assert torch.equal(yp, y[perm])
    assert torch.equal(dxp, dx[perm])
    assert rel_l2(to_np(dprojp[: min(E, 4)]), to_np(dproj[: min(E, 4)])) <= 4e-3  # same sums, other row order
    del yp, dxp, dfcp, dprojp

    # Oracle on a sample of tokens, forward and backward, routing tied to the GPU's logits.  Only the experts
    # that the sampled tokens selected are copied to the host; the logits are cut to those columns, which
    # leaves the top-k set, its order and the softmax unchanged.
    idx = torch.randperm(T, generator=torch.Generator().manual_seed(7))[: cfg["sample"]].to(DEV)
    lg = logits[idx]
    used = torch.unique(torch.topk(lg.float(), k, dim=-1).indices)
    _, osel_full, _ = O.topk_softmax(to_np(lg), k, "bf16")
    used = torch.from_numpy(np.unique(np.concatenate([to_np(used), osel_full.reshape(-1)]))).to(DEV)
    gate_w = moe.gate.weight[used]
    fwd = O.moe_forward(to_np(x[idx]), to_np(gate_w), to_np(moe.c_fc.weight[used]), to_np(moe.c_proj.weight[used]), k,
                        "bf16", logits=to_np(lg[:, used]))
    np.testing.assert_array_equal(to_np(used)[fwd["selected"]], osel_full)
    assert rel_l2(to_np(y[idx]), fwd["y"]) <= 1e-2
    bwd = O.moe_backward(fwd, to_np(dy[idx]), router_path=False)
    # dx of the layer = expert path + router path; the router path needs d_logits of these tokens only
    d_logits = O.topk_softmax_backward(fwd["softmax"], bwd["d_weights"], fwd["selected"], used.numel(), "bf16")
    want_dx = O.bf16_round(bwd["dx_experts"] + O.bf16_round(d_logits @ to_np(gate_w)))
    assert rel_l2(to_np(dx[idx]), want_dx) <= 1e-2

    # Weight gradients of single experts: the oracle as a one-expert layer over all rows of that expert,
    # with the routing weight folded into the upstream gradient (d_out = round(w * dy) either way).
    order = np.argsort(cnt, kind="stable")
    nonempty = order[cnt[order] > 0]
    picks = {int(nonempty[-1]), int(nonempty[0])}  # most and least loaded
    if E > 8:
        picks.add(int(nonempty[len(nonempty) // 2]))
    off = to_np(maps.pad_offsets)
    for e in sorted(picks):
        n = int(cnt[e])
        sl = maps.slot_of_row[int(off[e]) : int(off[e]) + n].long()
        tok, j = sl // k, sl % k
        w_rows, sel_rows, _ = O.topk_softmax(to_np(logits[tok]), k, "bf16")
        jj = to_np(j)
        assert np.all(sel_rows[np.arange(n), jj] == e)
        gate_col = w_rows[np.arange(n), jj][:, None]
        one = O.moe_forward(to_np(x[tok]), np.zeros((1, H), np.float32), to_np(moe.c_fc.weight[e : e + 1]),
                            to_np(moe.c_proj.weight[e : e + 1]), 1, "bf16", logits=np.zeros((n, 1), np.float32))
        grads = O.moe_backward(one, O.bf16_round(to_np(dy[tok]) * gate_col), router_path=False)
        assert rel_l2(to_np(dfc[e]), grads["d_w_fc"][0]) <= 1e-2, (e, n)
        assert rel_l2(to_np(dproj[e]), grads["d_w_proj"][0]) <= 1e-2, (e, n)
