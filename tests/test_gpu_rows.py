"""Token scatter / weighted combine and their backward passes on the GPU against numpy."""

import numpy as np
import pytest
import torch

from _util import DEV, TOL, randn, rel_l2, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

CASES = [(1, 8, 2, 1), (7, 64, 4, 2), (130, 96, 6, 3), (1000, 256, 128, 8), (513, 1024, 8, 2)]


def _maps(T, E, k, seed):
    from fma_b200.modules import _kernels as K

    g = torch.Generator().manual_seed(seed)
    sel = torch.randint(0, E, (T, k), generator=g)
    return K.moe_sort(sel.to(DEV), E), O.row_maps(sel.numpy(), E, K.ROW_ALIGN)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,k", CASES)
def test_scatter_and_backward(dtype, T, H, E, k):
    from fma_b200.modules import _kernels as K

    maps, ref = _maps(T, E, k, seed=T + H)
    x = randn((T, H), dtype, seed=1)
    grouped = K.scatter(x.to(DEV), maps)
    total = int(ref["pad_offsets"][-1])
    want = np.zeros((total, H), np.float32)
    valid = ref["slot_of_row"][:total] >= 0
    want[valid] = to_np(x)[ref["slot_of_row"][:total][valid] // k]
    np.testing.assert_array_equal(to_np(grouped)[:total], want)  # pure copy + zero padding: exact

    d_grouped = randn((maps.rows_cap, H), dtype, seed=2)
    dx = K.scatter_backward(d_grouped.to(DEV), maps, T)
    rows = ref["row_of_slot"].reshape(T, k)
    want_dx = to_np(d_grouped)[rows].astype(np.float64).sum(1)
    assert rel_l2(to_np(dx), want_dx) <= (TOL[dtype] if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,k", CASES)
def test_combine_and_backward(dtype, T, H, E, k):
    from fma_b200.modules import _kernels as K

    maps, ref = _maps(T, E, k, seed=T + H + 1)
    out = randn((maps.rows_cap, H), dtype, seed=3)
    w = torch.softmax(randn((T, k), torch.float32, seed=4), -1).to(dtype)
    dy = randn((T, H), dtype, seed=5)
    rows = ref["row_of_slot"].reshape(T, k)
    y = K.combine(out.to(DEV), w.to(DEV), maps, T)
    want_y = (to_np(out)[rows].astype(np.float64) * to_np(w)[:, :, None]).sum(1)
    assert rel_l2(to_np(y), want_y) <= (TOL[dtype] if dtype == torch.float32 else 4e-3)

    d_out, d_w = K.combine_backward(dy.to(DEV), out.to(DEV), w.to(DEV), maps)
    total = int(ref["pad_offsets"][-1])
    want_d_out = np.zeros((total, H), np.float64)
    want_d_out[rows.reshape(-1)] = (to_np(w).reshape(-1, 1).astype(np.float64) * np.repeat(to_np(dy), k, 0))
    got = to_np(d_out)[:total]
    assert rel_l2(got, want_d_out) <= (TOL[dtype] if dtype == torch.float32 else 4e-3)
    pad = ref["slot_of_row"][:total] < 0
    assert np.all(got[pad] == 0)  # padding rows must be exactly zero (they feed the weight-gradient GEMMs)
    want_d_w = (to_np(out)[rows].astype(np.float64) * to_np(dy)[:, None, :]).sum(-1)
    assert rel_l2(to_np(d_w), want_d_w) <= (TOL[dtype] if dtype == torch.float32 else 6e-3)

    # deterministic: same bits on a second run
    y2 = K.combine(out.to(DEV), w.to(DEV), maps, T)
    assert torch.equal(y, y2)
