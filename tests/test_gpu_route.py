"""Router top-k/softmax and the expert sort on the GPU against the CPU oracle.  Index results are
bit-exact; softmax weights are compared within the float tolerance of the dtype."""

import numpy as np
import pytest
import torch

from _util import DEV, ORACLE_DTYPE, TOL, randn, rel_l2, to_np, zipf_ids
from oracle import int_oracle
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,k", [(1, 2, 1), (7, 8, 2), (129, 6, 3), (1000, 128, 8), (333, 1000, 4), (64, 33, 32), (50, 4, 1)])
def test_topk_softmax_matches_oracle(dtype, T, E, k):
    from fma_b200.modules import _kernels as K

    logits = randn((T, E), dtype, seed=T + E + k)  # bf16 logits contain ties; the rule is lowest id first
    w, sel = K.router_topk_softmax(logits.to(DEV), k)
    ow, osel, _ = O.topk_softmax(to_np(logits), k, ORACLE_DTYPE[dtype])
    np.testing.assert_array_equal(to_np(sel), osel)
    assert rel_l2(to_np(w), ow) <= TOL[dtype]
    assert np.allclose(to_np(w).sum(-1), 1.0, atol=2e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_softmax_backward_matches_oracle(dtype):
    from fma_b200.modules import _kernels as K

    T, E, k = 257, 64, 6
    logits = randn((T, E), dtype, seed=1)
    d_w = randn((T, k), dtype, seed=2)
    w, sel = K.router_topk_softmax(logits.to(DEV), k)
    d_logits = K.router_topk_softmax_backward(w, d_w.to(DEV), sel, E)
    _, osel, p = O.topk_softmax(to_np(logits), k, ORACLE_DTYPE[dtype])
    want = O.topk_softmax_backward(p, to_np(d_w), osel, E, ORACLE_DTYPE[dtype])
    assert rel_l2(to_np(d_logits), want) <= (1e-5 if dtype == torch.float32 else 1e-2)
    mask = np.ones((T, E), bool)
    np.put_along_axis(mask, osel, False, -1)
    assert np.all(to_np(d_logits)[mask] == 0)


def _check_sort(sel: torch.Tensor, E: int, align: int = 128):
    from fma_b200.modules import _kernels as K

    maps = K.moe_sort(sel.to(DEV), E, want_sorted=True, row_align=align)
    ref = int_oracle.sort_maps(sel.numpy(), E, align)
    ref2 = O.row_maps(sel.numpy(), E, align)
    st_e, st_s = torch.sort(sel.flatten(), stable=True)
    np.testing.assert_array_equal(to_np(maps.sorted_expert_idxs), st_e.numpy())
    np.testing.assert_array_equal(to_np(maps.sorted_scattered_idxs), st_s.numpy())
    np.testing.assert_array_equal(to_np(maps.expert_count), torch.bincount(sel.flatten(), minlength=E).numpy())
    assert maps.rows_cap == ref["rows_cap"] == ref2["rows_cap"]
    for key in ("expert_count", "pad_offsets", "row_of_slot", "slot_of_row"):
        np.testing.assert_array_equal(to_np(getattr(maps, key)), ref[key].astype(np.int64), err_msg=key)
    if align % 128 == 0:
        np.testing.assert_array_equal(to_np(maps.mtile_expert), ref["mtile_expert"])
    return maps


@pytest.mark.parametrize("T,E,k", [(1, 1, 1), (1, 2, 1), (7, 8, 2), (127, 6, 3), (128, 6, 3), (129, 6, 3), (4096, 8, 2),
                                   (5000, 128, 8), (3001, 1000, 3), (100000, 128, 8)])
def test_sort_uniform(T, E, k):
    g = torch.Generator().manual_seed(T * 31 + E)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(min(T, 64))])
    if T > 64:  # cheaper generator for big cases: independent draws (duplicates within a row are legal ids)
        sel = torch.randint(0, E, (T, k), generator=g)
    _check_sort(sel, E)


def test_sort_skewed_with_empty_experts():
    T, E, k = 32768, 128, 8
    sel = zipf_ids(T * k, E, 1.0, seed=9, dtype=torch.int64).view(T, k)
    sel[sel == 5] = 6
    sel[sel == 127] = 0
    maps = _check_sort(sel, E)
    cnt = to_np(maps.expert_count)
    assert cnt[5] == 0 and cnt[127] == 0 and cnt.sum() == T * k


def test_sort_all_to_one_expert_and_unpadded():
    sel = torch.full((1000, 2), 3, dtype=torch.int64)
    _check_sort(sel, 8)
    g = torch.Generator().manual_seed(5)
    _check_sort(torch.randint(0, 16, (999, 4), generator=g), 16, align=1)
    _check_sort(torch.randint(0, 16, (999, 4), generator=g), 16, align=256)


def test_sort_is_deterministic():
    from fma_b200.modules import _kernels as K

    sel = torch.randint(0, 64, (20000, 4), generator=torch.Generator().manual_seed(1)).to(DEV)
    a = K.moe_sort(sel, 64, want_sorted=True)
    b = K.moe_sort(sel, 64, want_sorted=True)
    for key in ("sorted_scattered_idxs", "row_of_slot", "slot_of_row", "mtile_expert"):
        assert torch.equal(getattr(a, key), getattr(b, key))
