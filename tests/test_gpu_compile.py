"""The op surface under torch.compile(fullgraph=True), as the reference tests every op
(tests/ops/continuous_count_test.py:25, swiglu_test.py, grouped_gemm_test.py:25): the kernels are
registered as torch.library custom ops, so the compiler traces through the wrappers."""

import pytest
import torch

from _util import DEV, randn

pytestmark = pytest.mark.gpu


def test_continuous_count_compiled():
    import fma_b200

    fn = torch.compile(fma_b200.continuous_count, fullgraph=True)
    ids = torch.randint(0, 72, (16393,), generator=torch.Generator().manual_seed(1))
    for dtype in (torch.int32, torch.int64):
        got = fn(ids.to(dtype).to(DEV), 72)
        assert got.dtype == torch.uint32
        assert torch.equal(got.to(torch.int64).cpu(), torch.bincount(ids, minlength=72))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_compiled_forward_backward(dtype):
    import fma_b200

    gate = randn((257, 264), dtype, 1, 3.0).to(DEV).requires_grad_(True)
    up = randn((257, 264), dtype, 2).to(DEV).requires_grad_(True)
    dy = randn((257, 264), dtype, 3).to(DEV)
    y = fma_b200.swiglu(gate, up)
    y.backward(dy)
    want = (y.detach().clone(), gate.grad.clone(), up.grad.clone())
    gate.grad = up.grad = None
    yc = torch.compile(fma_b200.swiglu, fullgraph=True)(gate, up)
    yc.backward(dy)
    assert torch.equal(yc, want[0]) and torch.equal(gate.grad, want[1]) and torch.equal(up.grad, want[2])

    x = torch.cat([up.detach(), gate.detach()], -1).requires_grad_(True)
    yp = torch.compile(fma_b200.swiglu_packed, fullgraph=True)(x)
    yp.backward(dy)
    assert torch.equal(yp, want[0])
    assert torch.equal(x.grad, torch.cat([want[2], want[1]], -1))


def test_grouped_gemm_compiled():
    import fma_b200

    Ms, N, Kd = [256, 72, 0, 136], 264, 192
    g = torch.Generator().manual_seed(3)
    As = [torch.randint(-8, 9, (m, Kd), generator=g).to(torch.bfloat16) for m in Ms]
    Bs = [torch.randint(-8, 9, (N, Kd), generator=g).to(torch.bfloat16) for _ in Ms]
    A = torch.cat([a.reshape(-1) for a in As]).to(DEV)
    B = torch.cat([b.reshape(-1) for b in Bs]).to(DEV)
    u32 = lambda v: torch.tensor(v, dtype=torch.uint32, device=DEV)  # noqa: E731
    fn = torch.compile(fma_b200.grouped_gemm, fullgraph=True)
    out = fn(A=A, B=B, C=None, M_array=u32(Ms), N_array=u32([N] * 4), K_array=u32([Kd] * 4),
             output_shape=(sum(Ms) * N,), is_A_transposed=False, is_B_transposed=True)
    want = torch.cat([(a.float() @ b.float().T).to(torch.bfloat16).reshape(-1) for a, b in zip(As, Bs)])
    assert torch.equal(out.cpu(), want)


def test_moe_layer_compiled_fullgraph():
    """The whole layer under torch.compile(fullgraph=True), forward and backward, as the reference compiles
    its MoE (tests/modules/moe_test.py:97-98): same kernels in the same order as the eager path."""
    import fma_b200
    from fma_b200 import _native

    T, H, E, k, I = 384, 256, 8, 2, 128
    dtype = torch.bfloat16
    moe = fma_b200.MoE(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02)
    with torch.no_grad():
        moe.gate.weight.copy_(randn((E, H), torch.float32, 1, 0.02))
        moe.c_fc.weight.copy_(randn((E, 2 * I, H), torch.float32, 2, 0.02))
        moe.c_proj.weight.copy_(randn((E, H, I), torch.float32, 3, 0.02))
    moe = moe.to(DEV).to(dtype)
    x = randn((3, T // 3, H), dtype, 4).to(DEV)
    g = randn((3, T // 3, H), dtype, 5).to(DEV)

    def run(fn):
        for p in moe.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        y, logits = fn(xi)
        y.backward(g)
        return [y.detach(), logits.detach(), xi.grad] + [p.grad.clone() for p in moe.parameters()]

    eager = run(moe)
    compiled = run(torch.compile(moe, fullgraph=True))
    assert _native.device_status() == 0
    assert compiled[0].shape == x.shape and compiled[1].shape == (T, E)
    if torch.equal(eager[1], compiled[1]):  # same logits -> same routing -> same kernels on the same data
        for a, b in zip(eager, compiled):
            assert torch.equal(a, b)
    else:  # the compiler chose another GEMM for the router: near-ties may route differently
        for a, b in zip(eager, compiled):
            assert float((a.float() - b.float()).norm() / b.float().norm()) <= 1e-2


@pytest.mark.parametrize("case", ["gelu", "glu", "swiglu_bias"])
def test_moe_layer_compiled_fullgraph_other_experts(case):
    """torch.compile(fullgraph=True) of layers whose experts do not take the fused SwiGLU path: a non-gated
    tanh-GELU, torch's GLU (the two activations of the reference's MoE test, tests/test_commons.py:85-86) and
    SwiGLU experts with bias.  The activation is traced as ordinary code between two expert-linear ops."""
    import torch.nn.functional as F

    import fma_b200
    from fma_b200 import _native

    T, H, E, k, I = 384, 256, 8, 2, 128
    dtype = torch.bfloat16
    act, is_glu, bias = {
        "gelu": (lambda t: F.gelu(t, approximate="tanh"), False, False),
        "glu": (lambda t: F.glu(t, dim=-1), True, False),
        "swiglu_bias": (fma_b200.swiglu_packed, True, True),
    }[case]
    moe = fma_b200.MoE(E, k, H, I, act, is_glu, bias, 0.02)
    with torch.no_grad():
        moe.gate.weight.copy_(randn((E, H), torch.float32, 1, 0.02))
        moe.c_fc.weight.copy_(randn(tuple(moe.c_fc.weight.shape), torch.float32, 2, 0.02))
        moe.c_proj.weight.copy_(randn((E, H, I), torch.float32, 3, 0.02))
        if bias:
            moe.c_fc.bias.copy_(randn(tuple(moe.c_fc.bias.shape), torch.float32, 6, 0.1))
            moe.c_proj.bias.copy_(randn((E, H), torch.float32, 7, 0.1))
    moe = moe.to(DEV).to(dtype)
    x = randn((T, H), dtype, 4).to(DEV)
    g = randn((T, H), dtype, 5).to(DEV)

    def run(fn):
        for p in moe.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        y, logits = fn(xi)
        y.backward(g)
        return [y.detach(), logits.detach(), xi.grad] + [p.grad.clone() for p in moe.parameters()]

    eager = run(moe)
    compiled = run(torch.compile(moe, fullgraph=True))
    assert _native.device_status() == 0
    for a, b in zip(eager, compiled):
        assert a.shape == b.shape
        assert float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)) <= 1e-2
