"""Grouped GEMMs on the GPU.

bf16 (tcgen05 kernel): integer-valued operands make fp32 accumulation exact, so results must equal
the bf16 rounding of the exact product bit for bit (the known-answer design of the reference's
tests/ops/grouped_gemm_test.py:43-92).  fp32 (FFMA kernel): rel-L2 <= 1e-5 against float64.
"""

import numpy as np
import pytest
import torch

from _util import DEV, check_device_status, randn, rel_l2, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _int_tensor(shape, seed, lo=-8, hi=9, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g).to(dtype)


def _layer_maps(counts, E, row_align=256):
    """Row maps for given per-expert token counts (k = 1: slot == token).  row_align 256 runs the
    CTA-pair kernels (cta_group::2), 128 the single-CTA kernels."""
    from fma_b200.modules import _kernels as K

    sel = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    sel = sel[torch.randperm(sel.numel(), generator=torch.Generator().manual_seed(1))].view(-1, 1)
    return K.moe_sort(sel.to(DEV), E, row_align=row_align), sel


def _segments(maps):
    off = to_np(maps.pad_offsets)
    cnt = to_np(maps.expert_count)
    return off, cnt


LAYER_SHAPES = [
    # counts per expert, OUT, IN
    ([128, 256], 256, 64),
    ([5, 0, 300, 129], 512, 128),
    ([1000, 3, 0, 0, 77, 640], 264, 200),   # OUT, IN not multiples of the tile
    ([200] * 16, 1024, 512),
]


@pytest.mark.parametrize("row_align", [128, 256])
@pytest.mark.parametrize("counts,OUT,IN", LAYER_SHAPES)
def test_bf16_forward_dgrad_wgrad_exact(counts, OUT, IN, row_align):
    from fma_b200.modules import _kernels as K

    E = len(counts)
    maps, _ = _layer_maps(counts, E, row_align)
    off, cnt = _segments(maps)
    rows = maps.rows_cap
    X = torch.zeros(rows, IN, dtype=torch.bfloat16)
    dY = torch.zeros(rows, OUT, dtype=torch.bfloat16)
    for e in range(E):  # token rows hold integers, padding rows stay zero as the layer guarantees
        X[off[e] : off[e] + cnt[e]] = _int_tensor((cnt[e], IN), 10 + e)
        dY[off[e] : off[e] + cnt[e]] = _int_tensor((cnt[e], OUT), 50 + e, -4, 5)
    W = _int_tensor((E, OUT, IN), 99, -4, 5)
    Xd, dYd, Wd = X.to(DEV), dY.to(DEV), W.to(DEV)

    Y = K.gemm_forward(Xd, Wd, maps.mtile_expert, row_align)
    dX = K.gemm_dgrad(dYd, Wd, maps.mtile_expert, row_align)
    dW = K.gemm_wgrad(dYd, Xd, E, maps.pad_offsets)
    check_device_status()
    for e in range(E):
        s, t = off[e], off[e + 1]
        want = (X[s:t].float() @ W[e].float().T).to(torch.bfloat16)
        assert torch.equal(Y[s:t].cpu(), want), f"forward, expert {e}"
        want = (dY[s:t].float() @ W[e].float()).to(torch.bfloat16)
        assert torch.equal(dX[s:t].cpu(), want), f"dgrad, expert {e}"
        want = (dY[s:t].float().T @ X[s:t].float()).to(torch.bfloat16)
        assert torch.equal(dW[e].cpu(), want), f"wgrad, expert {e}"


@pytest.mark.parametrize("row_align", [128, 256])
@pytest.mark.parametrize("counts,I,IN", [([128, 256], 128, 64), ([5, 0, 300, 129], 256, 128), ([333, 100, 1], 200, 72)])
def test_bf16_swiglu_epilogues(counts, I, IN, row_align):
    """Fused up-projection + SwiGLU and fused dgrad + SwiGLU backward against the unfused kernels."""
    from fma_b200.modules import _kernels as K

    E = len(counts)
    H = IN
    maps, _ = _layer_maps(counts, E, row_align)
    off, cnt = _segments(maps)
    rows = maps.rows_cap
    X = torch.zeros(rows, IN, dtype=torch.bfloat16)
    dOut = torch.zeros(rows, H, dtype=torch.bfloat16)
    for e in range(E):
        X[off[e] : off[e] + cnt[e]] = randn((cnt[e], IN), torch.bfloat16, 10 + e)
        dOut[off[e] : off[e] + cnt[e]] = randn((cnt[e], H), torch.bfloat16, 30 + e)
    Wfc = randn((E, 2 * I, IN), torch.bfloat16, 7, 0.2)
    Wproj = randn((E, H, I), torch.bfloat16, 8, 0.2)
    Xd, Wfcd, Wprojd, dOutd = X.to(DEV), Wfc.to(DEV), Wproj.to(DEV), dOut.to(DEV)

    pre, act = K.gemm_forward_swiglu(Xd, Wfcd, maps.mtile_expert, row_align=row_align)
    pre_ref = K.gemm_forward(Xd, Wfcd, maps.mtile_expert, 128)  # single-CTA kernel as the cross-check
    total = off[-1]
    assert torch.equal(pre[:total], pre_ref[:total])  # same accumulation, same rounding
    act_ref = O.swiglu_packed(to_np(pre_ref[:total]), "bf16")
    assert rel_l2(to_np(act[:total]), act_ref) <= 4e-3
    pad = to_np(maps.slot_of_row)[:total] < 0
    assert np.all(to_np(act[:total])[pad] == 0) and np.all(to_np(pre[:total])[pad] == 0)

    # a caller that keeps no `pre` (inference) gets the same act from the one-phase form of the epilogue
    none, act_only = K.gemm_forward_swiglu(Xd, Wfcd, maps.mtile_expert, keep_pre=False, row_align=row_align)
    assert none is None and torch.equal(act_only[:total], act[:total])

    d_pre = K.gemm_dgrad_swiglu(dOutd, Wprojd, pre, maps.mtile_expert, row_align)
    d_act = K.gemm_dgrad(dOutd, Wprojd, maps.mtile_expert, 128)
    gg, ug = O.swiglu_backward(to_np(pre[:total, I:]), to_np(pre[:total, :I]), to_np(d_act[:total]), "bf16")
    assert rel_l2(to_np(d_pre[:total, :I]), ug) <= 4e-3
    assert rel_l2(to_np(d_pre[:total, I:]), gg) <= 4e-3
    assert np.all(to_np(d_pre[:total])[pad] == 0)
    check_device_status()


@pytest.mark.parametrize("a_t", [False, True])
@pytest.mark.parametrize("b_t", [False, True])
def test_bf16_general_known_answer_reference_shapes(a_t, b_t):
    """The reference's own grouped_gemm test case: E=16, K=4096, N=512, ragged M summing to 65536."""
    from fma_b200 import grouped_gemm

    E, Kd, N = 16, 4096, 512
    Ms = [512, 3176, 2048] * 5 + [36856]
    M_array = torch.tensor(Ms, device=DEV, dtype=torch.uint32)
    N_array = torch.full_like(M_array, N)
    K_array = torch.full_like(M_array, Kd)
    g = torch.Generator(device=DEV).manual_seed(42)
    As = [torch.randint(-8, 9, (Kd, m) if a_t else (m, Kd), device=DEV, generator=g).to(torch.bfloat16) for m in Ms]
    Bs = [torch.randint(-8, 9, (N, Kd) if b_t else (Kd, N), device=DEV, generator=g).to(torch.bfloat16) for _ in Ms]
    A = torch.cat([a.view(-1) for a in As])
    B = torch.cat([b.view(-1) for b in Bs])
    out = grouped_gemm(A=A, B=B, C=None, M_array=M_array, N_array=N_array, K_array=K_array,
                       output_shape=(sum(Ms) * N,), is_A_transposed=a_t, is_B_transposed=b_t)
    check_device_status()
    D = torch.cat([((a.T if a_t else a).float() @ (b.T if b_t else b).float()).to(torch.bfloat16).view(-1)
                   for a, b in zip(As, Bs)])
    assert (out.float() - D.float()).abs().max().item() == 0


@pytest.mark.parametrize("a_t", [False, True])
@pytest.mark.parametrize("b_t", [False, True])
def test_bf16_general_ragged_everything(a_t, b_t):
    """Per-group M, N and K all differ; includes empty groups and sizes that are not tile multiples."""
    from fma_b200 import grouped_gemm

    Ms, Ns, Ks = [8, 0, 136, 264, 16], [16, 8, 264, 8, 520], [72, 64, 8, 200, 0]
    As = [_int_tensor((k, m) if a_t else (m, k), 1 + i) for i, (m, k) in enumerate(zip(Ms, Ks))]
    Bs = [_int_tensor((n, k) if b_t else (k, n), 20 + i) for i, (n, k) in enumerate(zip(Ns, Ks))]
    A = torch.cat([a.reshape(-1) for a in As]).to(DEV)
    B = torch.cat([b.reshape(-1) for b in Bs]).to(DEV)
    u32 = lambda v: torch.tensor(v, dtype=torch.uint32, device=DEV)  # noqa: E731
    out = grouped_gemm(A, B, None, u32(Ms), u32(Ns), u32(Ks), (sum(m * n for m, n in zip(Ms, Ns)),),
                       is_A_transposed=a_t, is_B_transposed=b_t)
    check_device_status()
    want = O.grouped_gemm(to_np(A), to_np(B), Ms, Ns, Ks, a_t, b_t, "bf16")
    np.testing.assert_array_equal(to_np(out), want)


@pytest.mark.parametrize("counts,OUT,IN", [([128, 256], 256, 64), ([5, 0, 300, 129], 512, 128), ([700, 3, 0, 90], 264, 200)])
def test_f32_forward_dgrad_wgrad(counts, OUT, IN):
    from fma_b200.modules import _kernels as K

    E = len(counts)
    maps, _ = _layer_maps(counts, E)
    off, cnt = _segments(maps)
    rows = maps.rows_cap
    X = torch.zeros(rows, IN)
    dY = torch.zeros(rows, OUT)
    for e in range(E):
        X[off[e] : off[e] + cnt[e]] = randn((cnt[e], IN), torch.float32, 10 + e)
        dY[off[e] : off[e] + cnt[e]] = randn((cnt[e], OUT), torch.float32, 50 + e)
    W = randn((E, OUT, IN), torch.float32, 99, 0.05)
    Y = K.gemm_forward(X.to(DEV), W.to(DEV), maps.mtile_expert)  # fp32 ignores the pairing
    dX = K.gemm_dgrad(dY.to(DEV), W.to(DEV), maps.mtile_expert)
    dW = K.gemm_wgrad(dY.to(DEV), X.to(DEV), E, maps.pad_offsets)
    for e in range(E):
        s, t = off[e], off[e + 1]
        if t > s:
            assert rel_l2(to_np(Y[s:t]), X[s:t].double() @ W[e].double().T) <= 1e-5 or cnt[e] == 0
            assert rel_l2(to_np(dX[s:t]), dY[s:t].double() @ W[e].double()) <= 1e-5 or cnt[e] == 0
        want = dY[s:t].double().T @ X[s:t].double()
        assert rel_l2(to_np(dW[e]), want) <= 1e-5


@pytest.mark.parametrize("counts,OUT,IN", [([256, 512], 512, 128), ([5, 0, 300, 129, 700], 520, 136),
                                           ([1000, 3, 0, 0, 77, 640], 264, 200), ([200] * 16, 1024, 512)])
def test_bf16_peer_store_epilogue_into_local_buffers(counts, OUT, IN):
    """The GEMMs that store every 128-row output tile at an address from a table (the expert-parallel
    return path) with a table that points into LOCAL memory: tiles in permuted order inside one buffer,
    every fifth tile in a second buffer.  The bits must equal the ordinary forward / dgrad.  Covers ragged
    counts, empty experts and widths that are not multiples of 64."""
    from fma_b200.modules import _kernels as K

    E = len(counts)
    maps, _ = _layer_maps(counts, E, 256)
    off, cnt = _segments(maps)
    rows = maps.rows_cap
    n_tiles = rows // 128
    used_tiles = off[-1] // 128
    X = torch.zeros(rows, IN, dtype=torch.bfloat16)
    dY = torch.zeros(rows, OUT, dtype=torch.bfloat16)
    for e in range(E):
        X[off[e] : off[e] + cnt[e]] = randn((cnt[e], IN), torch.bfloat16, 10 + e)
        dY[off[e] : off[e] + cnt[e]] = randn((cnt[e], OUT), torch.bfloat16, 50 + e)
    W = randn((E, OUT, IN), torch.bfloat16, 99, 0.1)
    Xd, dYd, Wd = X.to(DEV), dY.to(DEV), W.to(DEV)
    perm = torch.randperm(n_tiles, generator=torch.Generator().manual_seed(4)).tolist()
    for kind, width in (("forward", OUT), ("dgrad", IN)):
        ref = K.gemm_forward(Xd, Wd, maps.mtile_expert, 256) if kind == "forward" else \
            K.gemm_dgrad(dYd, Wd, maps.mtile_expert, 256)
        main = torch.full((n_tiles * 128, width), 7.0, dtype=torch.bfloat16, device=DEV)
        side = torch.full((n_tiles * 128, width), 7.0, dtype=torch.bfloat16, device=DEV)
        table = torch.empty(n_tiles, dtype=torch.int64)
        where = []
        for t in range(n_tiles):
            buf = side if t % 5 == 4 else main
            table[t] = buf.data_ptr() + perm[t] * 128 * width * 2
            where.append((buf, perm[t]))
        table_d = table.to(DEV)
        if kind == "forward":
            K.gemm_forward_peer(Xd, Wd, table_d, maps.mtile_expert, 256)
        else:
            K.gemm_dgrad_peer(dYd, Wd, table_d, maps.mtile_expert, 256)
        check_device_status()
        written = {id(main): set(), id(side): set()}
        for t in range(used_tiles):
            buf, slot = where[t]
            assert torch.equal(buf[slot * 128 : (slot + 1) * 128], ref[t * 128 : (t + 1) * 128]), (kind, t)
            written[id(buf)].add(slot)
        for buf in (main, side):  # nothing else was touched
            for slot in range(n_tiles):
                if slot not in written[id(buf)]:
                    assert torch.all(buf[slot * 128 : (slot + 1) * 128] == 7.0), (kind, slot)
