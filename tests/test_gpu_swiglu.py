"""swiglu / swiglu_packed on the GPU against the reference-generated golden vectors and the oracle."""

import numpy as np
import pytest
import torch

from _util import DEV, ORACLE_DTYPE, randn, rel_l2, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

# fp32: the reference's own test uses atol 5.5e-6 (tests/ops/swiglu_test.py:44-46); bf16: one rounding
TOL_SW = {torch.float32: 2e-6, torch.bfloat16: 4e-3}


@pytest.mark.parametrize("tag,dtype", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_golden(golden_dir, tag, dtype):
    from fma_b200 import swiglu, swiglu_packed

    z = np.load(golden_dir / "swiglu.npz")
    gate = torch.from_numpy(z[f"{tag}_gate"]).to(dtype).to(DEV).requires_grad_(True)
    up = torch.from_numpy(z[f"{tag}_up"]).to(dtype).to(DEV).requires_grad_(True)
    dy = torch.from_numpy(z[f"{tag}_dy"]).to(dtype).to(DEV)
    y = swiglu(gate, up)
    y.backward(dy)
    assert rel_l2(to_np(y), z[f"{tag}_y"]) <= TOL_SW[dtype]
    assert rel_l2(to_np(gate.grad), z[f"{tag}_gate_grad"]) <= TOL_SW[dtype]
    assert rel_l2(to_np(up.grad), z[f"{tag}_up_grad"]) <= TOL_SW[dtype]
    xp = torch.cat([up.detach(), gate.detach()], -1).requires_grad_(True)
    yp = swiglu_packed(xp)
    yp.backward(dy)
    assert rel_l2(to_np(yp), z[f"{tag}_y_packed"]) <= TOL_SW[dtype]
    assert rel_l2(to_np(xp.grad), np.concatenate([z[f"{tag}_up_grad"], z[f"{tag}_gate_grad"]], -1)) <= TOL_SW[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 8), (3, 5, 16), (257, 264), (2049, 1032)])
def test_against_oracle(dtype, shape):
    from fma_b200 import swiglu

    gate = randn(shape, dtype, 1, scale=4.0).to(DEV).requires_grad_(True)
    up = randn(shape, dtype, 2).to(DEV).requires_grad_(True)
    dy = randn(shape, dtype, 3).to(DEV)
    y = swiglu(gate, up)
    y.backward(dy)
    od = ORACLE_DTYPE[dtype]
    assert rel_l2(to_np(y), O.swiglu(to_np(gate), to_np(up), od)) <= TOL_SW[dtype]
    gg, ug = O.swiglu_backward(to_np(gate), to_np(up), to_np(dy), od)
    assert rel_l2(to_np(gate.grad), gg) <= TOL_SW[dtype]
    assert rel_l2(to_np(up.grad), ug) <= TOL_SW[dtype]


def test_extreme_gate_values_stay_finite():
    from fma_b200 import swiglu

    gate = torch.tensor([[-1e4, -100.0, -88.5, 0.0, 88.5, 100.0, 1e4, 3.0]], device=DEV)
    up = torch.ones_like(gate)
    y = swiglu(gate, up)
    assert torch.isfinite(y).all()
    np.testing.assert_allclose(to_np(y), O.swiglu(to_np(gate), to_np(up)), rtol=1e-6, atol=1e-30)
