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


# ---------------------------------------------------------------------------------------------
# NaN logits, the routed (fused) path, router statistics, ids outside the range
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_orders_nan_first_and_always_selects_valid_ids(dtype):
    """torch.topk (the reference) orders NaN as the largest value.  Rows with a few NaNs, with more NaNs
    than k, and of NaN only: the selected ids are k distinct ids in [0,E) and equal the oracle's, and the
    weights of a row that selected a NaN are NaN, as the reference's softmax makes them.  The kernel only
    writes ids, it never uses them as an index."""
    from fma_b200.modules import _kernels as K

    T, E, k = 64, 128, 8
    logits = randn((T, E), dtype, seed=3)
    logits[1, [5, 77, 100]] = float("nan")
    logits[2, :] = float("nan")
    logits[3, 10:30] = float("nan")
    logits[4, 0] = float("inf")
    logits[5, :] = float("-inf")
    logits[6, [0, 127]] = float("nan")
    w, sel = K.router_topk_softmax(logits.to(DEV), k)
    sel_np, w_np = to_np(sel), to_np(w)
    assert sel_np.min() >= 0 and sel_np.max() < E
    assert all(len(set(row)) == k for row in sel_np.tolist())
    ow, osel, _ = O.topk_softmax(to_np(logits), k, ORACLE_DTYPE[dtype])
    np.testing.assert_array_equal(sel_np, osel)
    np.testing.assert_array_equal(np.isnan(w_np), np.isnan(ow))
    assert np.isnan(w_np[[1, 2, 3, 6]]).all() and not np.isnan(w_np[7:]).any()
    good = ~np.isnan(ow).any(-1)
    assert rel_l2(w_np[good], ow[good]) <= TOL[dtype]
    # the sort accepts what the router produced
    maps = K.moe_sort(sel, E, want_sorted=True)
    np.testing.assert_array_equal(to_np(maps.expert_count), np.bincount(osel.reshape(-1), minlength=E))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,k", [(1, 2, 1), (7, 8, 2), (129, 6, 3), (1000, 128, 8), (333, 1000, 4), (64, 33, 32),
                                   (4096, 8, 2), (70000, 128, 8), (5000, 64, 5)])
def test_routed_path_equals_plain_topk_plus_sort(dtype, T, E, k):
    """router_topk_softmax_routed + moe_sort(routed_workspace=...) (histogram pass inside the top-k kernel)
    against the plain top-k, the plain sort and the oracle: all indices bit-exact."""
    from fma_b200.modules import _kernels as K
    from _util import check_device_status

    logits = randn((T, E), dtype, seed=T + 3 * E + k).to(DEV)
    w0, sel0 = K.router_topk_softmax(logits, k)
    w1, sel1, ws = K.router_topk_softmax_routed(logits, k, want_probs=True)
    assert torch.equal(sel0, sel1) and torch.equal(w0, w1)
    plain = K.moe_sort(sel0, E, want_sorted=True)
    routed = K.moe_sort(sel1, E, want_sorted=True, routed_workspace=ws, want_mean_prob=True)
    for key in ("sorted_expert_idxs", "sorted_scattered_idxs", "expert_count", "pad_offsets", "row_of_slot",
                "slot_of_row", "mtile_expert"):
        assert torch.equal(getattr(plain, key), getattr(routed, key)), key
    ref = O.row_maps(to_np(sel0), E, K.ROW_ALIGN)
    for key in ("expert_count", "pad_offsets", "row_of_slot", "slot_of_row", "mtile_expert"):
        np.testing.assert_array_equal(to_np(getattr(routed, key)), ref[key].astype(np.int64), err_msg=key)
    count, mean_prob = O.router_stats(to_np(logits), to_np(sel0), E)
    np.testing.assert_array_equal(to_np(routed.expert_count), count)
    assert rel_l2(to_np(routed.router_mean_prob), mean_prob) <= 2e-6  # fp32 sums of T probabilities
    again = K.moe_sort(sel1, E, routed_workspace=K.router_topk_softmax_routed(logits, k, want_probs=True)[2],
                       want_mean_prob=True)
    assert torch.equal(again.router_mean_prob, routed.router_mean_prob)  # fixed summation order
    check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mean_prob_backward_matches_oracle(dtype):
    from fma_b200.modules import _kernels as K

    T, E = 777, 96
    logits = randn((T, E), dtype, seed=11)
    g = randn((E,), torch.float32, seed=12)
    d_logits = K.router_mean_prob_backward(logits.to(DEV), g.to(DEV))
    want = O.mean_prob_backward(to_np(logits), to_np(g))
    assert rel_l2(to_np(d_logits), want) <= (1e-5 if dtype == torch.float32 else 6e-3)


def test_layer_load_balancing_loss_and_its_gradient():
    """MoE.load_balancing_loss() (E * sum_e f_e P_e from the routing kernels' by-products) against the
    oracle's restatement, and its gradient with respect to the gate weight against the analytic one."""
    import fma_b200

    T, H, E, k, I = 600, 64, 16, 4, 64
    moe = fma_b200.MoE(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02).to(DEV)
    moe.collect_router_stats = True
    x = randn((T, H), torch.float32, seed=5).to(DEV)
    y, logits = moe(x)
    loss = moe.load_balancing_loss()
    sel = to_np(moe.last_row_maps.row_of_slot)  # forces the maps to exist; ids come from the oracle below
    assert sel.size == T * k
    _, osel, _ = O.topk_softmax(to_np(logits), k, "f32")
    want = O.load_balancing_loss(to_np(logits), osel, E)
    assert abs(float(loss) - want) <= 1e-5 * abs(want)
    loss.backward()
    count, _ = O.router_stats(to_np(logits), osel, E)
    d_mean = E * count.astype(np.float64) / T
    d_logits = O.mean_prob_backward(to_np(logits), d_mean)
    want_gate = d_logits.T @ to_np(x).astype(np.float64)
    assert rel_l2(to_np(moe.gate.weight.grad), want_gate) <= 1e-4


def test_sort_skips_ids_outside_the_range_and_reports_them():
    """Ids -1 and E (and far outside) among valid ones: the sort records status 0x7003, counts and places
    the valid ids exactly as the oracle does for the valid subsequence, marks the others with row -1, and
    the row movers skip those slots."""
    from fma_b200 import _native
    from fma_b200.modules import _kernels as K

    T, E, k, H = 3000, 16, 4, 64
    g = torch.Generator().manual_seed(21)
    sel = torch.randint(0, E, (T, k), generator=g)
    bad = torch.rand(T, k, generator=g) < 0.01
    junk = torch.tensor([-1, E, E + 5, -(2**40), 2**40, 2**31])[torch.randint(0, 6, (T, k), generator=g)]
    sel = torch.where(bad, junk, sel)
    assert int(bad.sum()) > 20
    assert _native.device_status() == 0
    maps = K.moe_sort(sel.to(DEV), E, want_sorted=True)
    assert _native.device_status() == 0x7003
    assert _native.device_status() == 0  # reading clears the word
    flat = sel.flatten().numpy()
    ok = (flat >= 0) & (flat < E)
    np.testing.assert_array_equal(to_np(maps.expert_count), O.continuous_count(flat, E))
    ref = O.row_maps(flat[ok], E, K.ROW_ALIGN)  # the valid ids alone, in order
    row_of_slot = to_np(maps.row_of_slot)
    np.testing.assert_array_equal(row_of_slot[~ok], -1)
    np.testing.assert_array_equal(row_of_slot[ok], ref["row_of_slot"])
    np.testing.assert_array_equal(to_np(maps.pad_offsets), ref["pad_offsets"])
    n_ok = int(ok.sum())
    slots_ok = np.flatnonzero(ok)
    np.testing.assert_array_equal(to_np(maps.sorted_scattered_idxs)[:n_ok], slots_ok[ref["sorted_scattered_idxs"]])
    # scatter -> combine with unit weights through these maps: every token gets (valid slots) * x
    x = randn((T, H), torch.float32, seed=2).to(DEV)
    grouped = K.scatter(x, maps)
    w = torch.ones(T, k, device=DEV)
    y = K.combine(grouped, w, maps, T)
    n_valid = torch.from_numpy(ok.reshape(T, k).sum(1)).to(DEV)
    assert torch.allclose(y, x * n_valid[:, None].float(), rtol=1e-6, atol=1e-6)
    d_out, d_w = K.combine_backward(x, grouped, w, maps)
    assert torch.all(d_w[torch.from_numpy(~ok.reshape(T, k)).to(DEV)] == 0)
    dx = K.scatter_backward(d_out, maps, T)
    assert torch.allclose(dx, x * n_valid[:, None].float(), rtol=1e-6, atol=1e-6)
    assert _native.device_status() == 0
