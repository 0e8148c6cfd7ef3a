"""The layer at the full sizes of the benchmark configurations (Mixtral-shaped and fine-grained), where
the CPU oracle cannot evaluate the whole layer in seconds.  Checked through size-independent
properties, plus the oracle on a sample of tokens:
  * determinism: two runs give identical bits (no floating-point atomics anywhere);
  * token-permutation equivariance: y and dx follow a permutation of the tokens bit for bit, weight
    gradients keep their value up to summation order;
  * exact scaling: a backward pass with 2*dy gives exactly 2x every gradient (powers of two commute
    with every rounding step);
  * conservation: expert counts sum to T*k, every token slot owns exactly one grouped row;
  * sampled parity: for 48 sampled tokens the oracle (all experts, same logits) reproduces y.
"""

import numpy as np
import pytest
import torch

from _util import DEV, check_device_status, rel_l2, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

CONFIGS = {
    "mixtral_shaped": dict(T=16384, H=4096, E=8, k=2, I=14336, zipf=False),
    "fine_grained_zipf": dict(T=32768, H=2048, E=128, k=8, I=768, zipf=True),
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

    # oracle on a sample of tokens (all experts, routing tied to the GPU's logits)
    idx = torch.randperm(T, generator=torch.Generator().manual_seed(7))[:48].to(DEV)
    fwd = O.moe_forward(to_np(x[idx]), to_np(moe.gate.weight), to_np(moe.c_fc.weight), to_np(moe.c_proj.weight), k,
                        "bf16", logits=to_np(logits[idx]))
    assert rel_l2(to_np(y[idx]), fwd["y"]) <= 1e-2
