"""Pins the CPU oracle (oracle/) to the reference: every function is compared with vectors that
tests/golden/make_golden.py produced by running the reference's torch backend."""

import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import int_oracle
from oracle import moe_oracle as O

LAYER_CASES = ["layer_f32_small", "layer_f32_k1", "layer_bf16_small", "layer_bf16_many_experts"]


def _load(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz", allow_pickle=False)
    meta = json.loads(str(z["meta"]))
    return z, meta


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_matches_reference(golden_dir, name):
    z, meta = _load(golden_dir, name)
    dtype = "bf16" if "bfloat16" in meta["dtype"] else "f32"
    fwd = O.moe_forward(z["x"], z["w_gate"], z["w_fc"], z["w_proj"], meta["k"], dtype)
    assert O.rel_l2(fwd["router_logits"], z["router_logits"]) < (1e-6 if dtype == "f32" else 4e-3)
    if not np.array_equal(fwd["selected"], z["selected"]):
        # a differently rounded logit can only flip ties; feed the reference's logits instead
        fwd = O.moe_forward(z["x"], z["w_gate"], z["w_fc"], z["w_proj"], meta["k"], dtype, logits=z["router_logits"])
    # torch.topk does not promise an order among equal logits; compare as per-row sets when they tie
    sel_ref = z["selected"]
    same = np.array_equal(fwd["selected"], sel_ref)
    if not same:
        assert np.array_equal(np.sort(fwd["selected"], -1), np.sort(sel_ref, -1))
    np.testing.assert_array_equal(fwd["expert_count"], z["expert_count"])
    np.testing.assert_array_equal(fwd["sorted_expert_idxs"], z["stable_sorted_expert_idxs"])
    np.testing.assert_array_equal(fwd["sorted_expert_idxs"], z["ref_sorted_expert_idxs"])
    if same:
        np.testing.assert_array_equal(fwd["sorted_scattered_idxs"], z["stable_sorted_scattered_idxs"])
        # the reference's default sort is not stable: same rows per expert, maybe in another order
        off = fwd["offsets"]
        for e in range(len(off) - 1):
            a = np.sort(fwd["sorted_scattered_idxs"][off[e] : off[e + 1]])
            b = np.sort(z["ref_sorted_scattered_idxs"][off[e] : off[e + 1]])
            np.testing.assert_array_equal(a, b)
    bwd = O.moe_backward(fwd, z["g"])
    tol = 2e-6 if dtype == "f32" else 6e-3
    assert O.rel_l2(fwd["y"], z["y"]) < tol
    assert O.rel_l2(bwd["dx"], z["dx"]) < tol
    assert O.rel_l2(bwd["d_w_fc"], z["d_w_fc"]) < tol
    assert O.rel_l2(bwd["d_w_proj"], z["d_w_proj"]) < tol
    if meta["k"] > 1:
        assert O.rel_l2(bwd["d_w_gate"], z["d_w_gate"]) < (2e-5 if dtype == "f32" else 2e-2)
    else:
        assert np.abs(z["d_w_gate"]).max() == 0 and np.abs(bwd["d_w_gate"]).max() == 0


@pytest.mark.parametrize("name", ["layer_f32_bias", "layer_bf16_bias"])
def test_layer_with_expert_bias_matches_reference(golden_dir, name):
    z, meta = _load(golden_dir, name)
    dtype = "bf16" if "bfloat16" in meta["dtype"] else "f32"
    fwd = O.moe_forward(z["x"], z["w_gate"], z["w_fc"], z["w_proj"], meta["k"], dtype, logits=z["router_logits"],
                        b_fc=z["b_fc"], b_proj=z["b_proj"])
    assert np.array_equal(np.sort(fwd["selected"], -1), np.sort(z["selected"], -1))
    np.testing.assert_array_equal(fwd["expert_count"], z["expert_count"])
    bwd = O.moe_backward(fwd, z["g"])
    tol = 2e-6 if dtype == "f32" else 6e-3
    assert O.rel_l2(fwd["y"], z["y"]) < tol
    for key in ("dx", "d_w_fc", "d_w_proj", "d_b_fc", "d_b_proj"):
        assert O.rel_l2(bwd[key], z[key]) < tol, key


def test_layer_float16_matches_reference(golden_dir):
    """The oracle with IEEE-half rounding points against the reference run in float16 (the dtype the kernels
    of this repository do not cover yet: this pins the checker for it)."""
    z, meta = _load(golden_dir, "layer_f16_small")
    fwd = O.moe_forward(z["x"], z["w_gate"], z["w_fc"], z["w_proj"], meta["k"], "f16", logits=z["router_logits"])
    assert np.array_equal(np.sort(fwd["selected"], -1), np.sort(z["selected"], -1))
    np.testing.assert_array_equal(fwd["expert_count"], z["expert_count"])
    bwd = O.moe_backward(fwd, z["g"])
    assert O.rel_l2(fwd["y"], z["y"]) < 1e-3
    for key in ("dx", "d_w_fc", "d_w_proj"):
        assert O.rel_l2(bwd[key], z[key]) < 1e-3, key


def test_layer_config1_statistics(golden_dir):
    """The small fp32 configuration (T=4096, H=1024, E=8, top-2, I=512, seed 0) regenerated from its
    recipe and compared with the statistics the reference produced."""
    stats = json.loads((golden_dir / "layer_f32_config1_stats.json").read_text())
    torch.manual_seed(0)
    E, k, H, I = 8, 2, 1024, 512
    # parameter creation order of MoE.__init__: gate (nn.Linear), c_fc, c_proj; then gate re-drawn
    torch.nn.Linear(H, E, bias=False)
    w_fc = torch.empty(E, 2 * I, H).normal_(0, 0.02)
    w_proj = torch.empty(E, H, I).normal_(0, 0.02)
    w_gate = torch.empty(E, H).normal_(0, 0.02)
    x = torch.randn(4096, H)
    g = torch.randn(4096, H)
    fwd = O.moe_forward(x.numpy(), w_gate.numpy(), w_fc.numpy(), w_proj.numpy(), k, "f32")
    assert [int(v) for v in fwd["expert_count"]] == stats["expert_count"]
    assert [int(v) for v in fwd["expert_count"]] == [1065, 1035, 1107, 1007, 1021, 974, 1009, 974]
    for key, arr in (("selected", fwd["selected"]), ("stable_sorted_expert_idxs", fwd["sorted_expert_idxs"]),
                     ("stable_sorted_scattered_idxs", fwd["sorted_scattered_idxs"])):
        assert hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()[:16] == stats[key + "_sha16"]
    bwd = O.moe_backward(fwd, g.numpy())
    got = {"y": fwd["y"], "router_logits": fwd["router_logits"], "dx": bwd["dx"], "d_w_fc": bwd["d_w_fc"],
           "d_w_proj": bwd["d_w_proj"], "d_w_gate": bwd["d_w_gate"]}
    for key, arr in got.items():
        ref = stats[key]
        a = arr.astype(np.float64)
        assert abs(np.linalg.norm(a) - ref["l2"]) <= 2e-5 * ref["l2"], key
        sample = arr.reshape(-1)[:: max(1, arr.size // 64)][:64]
        np.testing.assert_allclose(sample, np.array(ref["sample"], dtype=np.float32), rtol=2e-4, atol=2e-5, err_msg=key)


def test_continuous_count_matches_reference(golden_dir):
    z = np.load(golden_dir / "continuous_count.npz")
    for i in range(int(z["n_cases"])):
        ids, size, ref = z[f"ids_{i}"], int(z[f"size_{i}"]), z[f"count_{i}"]
        np.testing.assert_array_equal(O.continuous_count(ids, size).astype(np.int64), ref)
        if size > 1:
            np.testing.assert_array_equal(int_oracle.count(ids, size).astype(np.int64), ref)


def test_count_ignores_out_of_range():
    ids = np.array([0, 5, -1, 3, 7, 3, 100], dtype=np.int32)
    np.testing.assert_array_equal(O.continuous_count(ids, 4), [1, 0, 0, 2])
    np.testing.assert_array_equal(int_oracle.count(ids, 4), [1, 0, 0, 2])


@pytest.mark.parametrize("R,E,align", [(0, 4, 128), (1, 1, 128), (1000, 7, 128), (5000, 128, 128), (300, 5, 1), (4096, 8, 256)])
def test_c_and_numpy_sort_maps_agree(R, E, align):
    rng = np.random.default_rng(R + E)
    sel = rng.integers(0, E, R).astype(np.int64)
    if E > 2 and R > 0:
        sel[sel == 1] = 0  # leave one expert empty
    a = O.row_maps(sel, E, align)
    b = int_oracle.sort_maps(sel, E, align)
    for key in ("sorted_expert_idxs", "sorted_scattered_idxs", "expert_count", "pad_offsets", "row_of_slot", "slot_of_row"):
        np.testing.assert_array_equal(a[key], b[key], err_msg=key)
    if align % 128 == 0:
        np.testing.assert_array_equal(a["mtile_expert"], b["mtile_expert"])
    ref_e, ref_s = torch.sort(torch.from_numpy(sel), stable=True)
    np.testing.assert_array_equal(a["sorted_expert_idxs"], ref_e.numpy())
    np.testing.assert_array_equal(a["sorted_scattered_idxs"], ref_s.numpy())


@pytest.mark.parametrize("tag,tol", [("f32", 1e-6), ("bf16", 4e-3)])
def test_swiglu_matches_reference(golden_dir, tag, tol):
    z = np.load(golden_dir / "swiglu.npz")
    gate, up, dy = z[f"{tag}_gate"], z[f"{tag}_up"], z[f"{tag}_dy"]
    assert O.rel_l2(O.swiglu(gate, up, tag), z[f"{tag}_y"]) < tol
    gg, ug = O.swiglu_backward(gate, up, dy, tag)
    assert O.rel_l2(gg, z[f"{tag}_gate_grad"]) < tol
    assert O.rel_l2(ug, z[f"{tag}_up_grad"]) < tol
    assert O.rel_l2(O.swiglu_packed(np.concatenate([up, gate], -1), tag), z[f"{tag}_y_packed"]) < tol


def test_grouped_gemm_known_answer():
    """Integer-valued operands make fp32 accumulation exact, so the packed result must equal A@B
    exactly (the design of the reference's tests/ops/grouped_gemm_test.py:43-92)."""
    rng = np.random.default_rng(3)
    M, N, K = [5, 0, 17, 8], [16, 16, 8, 24], [32, 32, 40, 8]
    for a_t in (False, True):
        for b_t in (False, True):
            As = [rng.integers(-8, 9, (k, m) if a_t else (m, k)).astype(np.float32) for m, k in zip(M, K)]
            Bs = [rng.integers(-8, 9, (n, k) if b_t else (k, n)).astype(np.float32) for n, k in zip(N, K)]
            got = O.grouped_gemm(np.concatenate([a.ravel() for a in As]), np.concatenate([b.ravel() for b in Bs]),
                                 M, N, K, a_t, b_t, "f32")
            want = np.concatenate([((a.T if a_t else a) @ (b.T if b_t else b)).ravel() for a, b in zip(As, Bs)])
            np.testing.assert_array_equal(got, want)


def test_bf16_round_matches_torch():
    x = torch.randn(10000) * 37
    want = x.to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(O.bf16_round(x.numpy()), want)


@pytest.mark.parametrize("side", ["left", "right"])
def test_sequence_packing_matches_reference(golden_dir, side):
    """pack_sequence / unpack_sequence of the oracle against the reference's torch backend (fixture generated
    by importing the reference): exact copies, zeros in the padding."""
    z = np.load(golden_dir / "sequence_packing.npz")
    np.testing.assert_array_equal(O.pack_sequence(z["padded"], z["cu_seqlens"], side), z[f"packed_{side}"])
    np.testing.assert_array_equal(O.unpack_sequence(z["packed_in"], z["cu_seqlens"], (5, 7, 2, 4), side),
                                  z[f"unpacked_{side}"])
