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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,k", CASES)
def test_expert_bias_add_and_grad(dtype, T, H, E, k):
    """grouped[p] += bias[e(p)] on token rows only (padding rows stay exactly zero), and the
    per-expert column sums that are the bias gradient."""
    from fma_b200.modules import _kernels as K

    maps, ref = _maps(T, E, k, seed=T + 3 * H)
    x = randn((T, H), dtype, seed=4)
    bias = randn((E, H), dtype, seed=5)
    grouped = K.scatter(x.to(DEV), maps)
    before = to_np(grouped).copy()
    K.bias_add_(grouped, bias.to(DEV), maps)
    total = int(ref["pad_offsets"][-1])
    slot = ref["slot_of_row"][:total]
    expert_of_row = np.repeat(np.arange(E), np.diff(ref["pad_offsets"]))
    want = before[:total].copy()
    valid = slot >= 0
    summed = (torch.from_numpy(before[:total][valid]) + torch.from_numpy(to_np(bias)[expert_of_row[valid]])).to(dtype)
    want[valid] = summed.float().numpy()
    np.testing.assert_array_equal(to_np(grouped)[:total], want)  # one rounded add per element: exact

    d = to_np(grouped)[:total].astype(np.float64)  # rows past the last segment are never written
    got = K.bias_grad(grouped, maps)
    want_g = np.stack([d[ref["pad_offsets"][e] : ref["pad_offsets"][e + 1]].sum(0) for e in range(E)])
    assert rel_l2(to_np(got), want_g) <= (1e-5 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("counts", [[5, 0, 300, 256], [1], [255, 257, 511, 0, 0, 3, 1024]])
def test_zero_padding_rows(dtype, counts):
    """fma_b200_moe_zero_padding: only the rows between the end of a segment's token rows and the start of the next
    segment are zeroed; token rows and everything past the last segment stay as they were."""
    from fma_b200.modules import _kernels as K

    align, H = 256, 72
    offs = [0]
    for n in counts:
        offs.append(offs[-1] + (n + align - 1) // align * align)
    base, extra = 3, 7  # the layout starts at row `base` of a larger buffer
    rows = torch.full((base + offs[-1] + extra, H), 1.5, dtype=dtype, device=DEV)
    seg = torch.tensor(offs, dtype=torch.int32, device=DEV)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    view = rows[base:]
    K.call("fma_b200_moe_zero_padding", K.ptr(view), H * rows.element_size(), K.ptr(seg), K.ptr(cnt), len(counts),
           K.stream_ptr(DEV))  # fmt: skip
    want = np.full((base + offs[-1] + extra, H), 1.5, dtype=np.float32)
    for j, n in enumerate(counts):
        want[base + offs[j] + n : base + offs[j + 1]] = 0
    np.testing.assert_array_equal(to_np(rows).astype(np.float32), want)
