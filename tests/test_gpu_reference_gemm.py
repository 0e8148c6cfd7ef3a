"""This library's grouped GEMM against the reference project's own CUDA kernel, run on the same GPU: the
reference's CUTLASS grouped GEMM compiled unmodified from its sources (baseline/build_reference_gemm.py)
and called through its stock entry point.  Integer-valued operands make fp32 accumulation exact, so the two
results must agree bit for bit (the known-answer design of the reference's tests/ops/grouped_gemm_test.py).
Skipped when the reference kernel has not been built (its sources are not part of this repository)."""

import sys
from pathlib import Path

import pytest
import torch

from _util import DEV

pytestmark = pytest.mark.gpu
sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "baseline"))


def _ref():
    import reference_gemm

    ok, why = reference_gemm.available()
    if not ok:
        pytest.skip(why)
    if torch.cuda.device_count() != 1:
        pytest.skip("the reference kernel is run by single-GPU jobs only")
    return reference_gemm


@pytest.mark.parametrize("a_t,b_t", [(False, True), (False, False), (True, False)])
def test_general_grouped_gemm_equals_reference_kernel(a_t, b_t):
    """The three transpose combinations the layer uses (forward NT, dgrad NN, wgrad TN) on the reference
    test's own ragged case: E=16, K=4096, N=512, M summing to 65536."""
    ref = _ref()
    from fma_b200 import grouped_gemm

    E, Kd, N = 16, 4096, 512
    Ms = [512, 3176, 2048] * 5 + [36856]
    u32 = lambda v: torch.tensor(v, device=DEV, dtype=torch.uint32)  # noqa: E731
    M_array, N_array, K_array = u32(Ms), u32([N] * E), u32([Kd] * E)
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.cat([torch.randint(-8, 9, (Kd, m) if a_t else (m, Kd), device=DEV, generator=g).to(torch.bfloat16).view(-1)
                   for m in Ms])
    B = torch.cat([torch.randint(-8, 9, (N, Kd) if b_t else (Kd, N), device=DEV, generator=g).to(torch.bfloat16).view(-1)
                   for _ in Ms])
    shape = (sum(Ms) * N,)
    want = ref.grouped_gemm(A, B, M_array, N_array, K_array, shape, a_t, b_t)
    got = grouped_gemm(A=A, B=B, C=None, M_array=M_array, N_array=N_array, K_array=K_array, output_shape=shape,
                       is_A_transposed=a_t, is_B_transposed=b_t)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_layer_gemms_equal_reference_kernel():
    """The layer's own forward / dgrad / wgrad kernels (padded grouped layout) against the reference kernel on
    the reference's unpadded layout, same integer data: expert segments must agree bit for bit."""
    ref = _ref()
    from fma_b200.modules import _kernels as K

    E, OUT, IN = 8, 512, 256
    counts = [300, 8, 1000, 129, 256, 5, 640, 77]  # no empty group: what the reference kernel does with K = 0 is not relied on
    sel = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    sel = sel[torch.randperm(sel.numel(), generator=torch.Generator().manual_seed(1))].view(-1, 1)
    maps = K.moe_sort(sel.to(DEV), E)
    off = maps.pad_offsets.tolist()
    g = torch.Generator(device=DEV).manual_seed(7)
    ri = lambda *shape, lo=-4, hi=5: torch.randint(lo, hi, shape, device=DEV, generator=g).to(torch.bfloat16)  # noqa: E731
    W = ri(E, OUT, IN)
    x_plain, dy_plain = ri(sum(counts), IN, lo=-8, hi=9), ri(sum(counts), OUT)
    X = torch.zeros(maps.rows_cap, IN, dtype=torch.bfloat16, device=DEV)
    dY = torch.zeros(maps.rows_cap, OUT, dtype=torch.bfloat16, device=DEV)
    start = 0
    for e, c in enumerate(counts):
        X[off[e] : off[e] + c] = x_plain[start : start + c]
        dY[off[e] : off[e] + c] = dy_plain[start : start + c]
        start += c
    u32 = lambda v: torch.tensor(v, device=DEV, dtype=torch.uint32)  # noqa: E731
    M_array, N_array, K_array = u32(counts), u32([OUT] * E), u32([IN] * E)
    y_ref = ref.grouped_gemm(x_plain, W, M_array, N_array, K_array, (sum(counts), OUT), False, True)
    dx_ref = ref.grouped_gemm(dy_plain, W, M_array, K_array, N_array, (sum(counts), IN), False, False)
    dw_ref = ref.grouped_gemm(dy_plain, x_plain, N_array, K_array, M_array, (E, OUT, IN), True, False)
    Y = K.gemm_forward(X, W, maps.mtile_expert)
    dX = K.gemm_dgrad(dY, W, maps.mtile_expert)
    dW = K.gemm_wgrad(dY, X, E, maps.pad_offsets)
    torch.cuda.synchronize()
    start = 0
    for e, c in enumerate(counts):
        assert torch.equal(Y[off[e] : off[e] + c], y_ref[start : start + c]), f"forward, expert {e}"
        assert torch.equal(dX[off[e] : off[e] + c], dx_ref[start : start + c]), f"dgrad, expert {e}"
        assert torch.equal(dW[e], dw_ref[e]), f"wgrad, expert {e}"
        start += c
