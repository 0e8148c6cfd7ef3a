"""The reference's own expert-linear entry points on its layout (expert e owns expert_frequency[e] consecutive
rows, no alignment): `grouped_gemm_experts` and `Experts.cuda_forward`
(fma/modules/moe/cuda_implementation/__init__.py:15-80, fma/modules/moe/__init__.py:89-92), forward and
backward, against per-expert matmuls on integer-valued operands (every product and sum is exact in bf16, the
design of the reference's grouped-GEMM test)."""

import pytest
import torch

from _util import DEV

pytestmark = pytest.mark.gpu


def _ints(shape, seed, lo=-2, hi=3):
    return torch.randint(lo, hi, shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


# the reference pads every expert's rows to a multiple of 8 before this call (group_with_padding)
@pytest.mark.parametrize("counts", [[24, 8, 0, 40], [16] * 8, [8, 56, 0, 0, 64, 32]])
def test_experts_cuda_forward_and_backward(counts):
    import fma_b200

    E, N, K = len(counts), 64, 32
    experts = fma_b200.Experts(E, K, N, add_bias=False, std=0.02)
    with torch.no_grad():
        experts.weight.copy_(_ints((E, N, K), 1))
    experts = experts.to(DEV).to(torch.bfloat16)
    x = _ints((sum(counts), K), 2).to(DEV).requires_grad_(True)
    dy = _ints((sum(counts), N), 3).to(DEV)
    freq = torch.tensor(counts, dtype=torch.uint32, device=DEV)

    y = experts.cuda_forward(x, freq)
    y.backward(dy)

    w = experts.weight.detach().float()
    xs, dys = x.detach().float().split(counts), dy.float().split(counts)
    want_y = torch.cat([xs[e] @ w[e].T for e in range(E)])
    want_dx = torch.cat([dys[e] @ w[e] for e in range(E)])
    want_dw = torch.stack([dys[e].T @ xs[e] for e in range(E)])
    assert torch.equal(y.float(), want_y)
    assert torch.equal(x.grad.float(), want_dx)
    assert torch.equal(experts.weight.grad.float(), want_dw)
