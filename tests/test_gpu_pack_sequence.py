"""pack_sequence / unpack_sequence on the GPU: exact copies against the oracle and the reference-generated
fixture, every dtype, both padding sides, cu_seqlens as uint32 / int32 / int64, gradients (each op's backward
is the other op), a list of inputs, and under torch.compile(fullgraph=True)."""

import numpy as np
import pytest
import torch

from _util import DEV, randn, to_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("side", ["left", "right"])
def test_reference_fixture(golden_dir, side):
    import fma_b200

    z = np.load(golden_dir / "sequence_packing.npz")
    cu = torch.from_numpy(z["cu_seqlens"]).to(DEV)
    packed = fma_b200.pack_sequence(torch.from_numpy(z["padded"]).to(DEV), cu, padding_side=side)
    np.testing.assert_array_equal(to_np(packed), z[f"packed_{side}"])
    unpacked = fma_b200.unpack_sequence(torch.from_numpy(z["packed_in"]).to(DEV), cu, (5, 7, 2, 4), padding_side=side)
    np.testing.assert_array_equal(to_np(unpacked), z[f"unpacked_{side}"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("index_dtype", [torch.uint32, torch.int32, torch.int64])
@pytest.mark.parametrize("side", ["left", "right"])
def test_reference_test_shapes_with_gradients(dtype, index_dtype, side):
    """The reference test's own case (tests/ops/pack_sequence_test.py:18-19): 7 sequences of up to 1000
    positions, rows of 12 x 14 elements."""
    import fma_b200

    size, lens = (7, 1000, 12, 14), [0, 70, 170, 295, 393, 412, 515, 691]
    cu = torch.tensor(lens, dtype=torch.int64).to(index_dtype).to(DEV)
    x = randn(size, dtype, 1).to(DEV).requires_grad_(True)
    packed = fma_b200.pack_sequence(x, cu, padding_side=side)
    want = O.pack_sequence(to_np(x), np.array(lens), side)
    assert packed.shape == want.shape
    np.testing.assert_array_equal(to_np(packed), want)
    g = randn(tuple(packed.shape), dtype, 2).to(DEV)
    packed.backward(g)
    np.testing.assert_array_equal(to_np(x.grad), O.unpack_sequence(to_np(g), np.array(lens), size, side))

    p = randn((lens[-1], 12, 14), dtype, 3).to(DEV).requires_grad_(True)
    unpacked = fma_b200.unpack_sequence(p, cu, size, padding_side=side)
    np.testing.assert_array_equal(to_np(unpacked), O.unpack_sequence(to_np(p), np.array(lens), size, side))
    g2 = randn(size, dtype, 4).to(DEV)
    unpacked.backward(g2)
    np.testing.assert_array_equal(to_np(p.grad), O.pack_sequence(to_np(g2), np.array(lens), side))


def test_lists_output_shape_and_round_trip():
    import fma_b200

    lens = [0, 5, 5, 12, 20]
    cu = torch.tensor(lens, dtype=torch.int32, device=DEV)
    a, b = randn((4, 8, 16), torch.float32, 1).to(DEV), randn((4, 8, 4, 8), torch.bfloat16, 2).to(DEV)
    pa, pb = fma_b200.pack_sequence([a, b], cu, padding_side="right")
    assert pa.shape == (20, 16) and pb.shape == (20, 4, 8)
    back = fma_b200.unpack_sequence(pa, cu, (4, 8, 16), padding_side="right")
    mask = torch.zeros(4, 8, dtype=torch.bool, device=DEV)
    for i in range(4):
        mask[i, : lens[i + 1] - lens[i]] = True
    assert torch.equal(back[mask], a[mask]) and torch.all(back[~mask] == 0)
    with pytest.raises(ValueError):
        fma_b200.pack_sequence(a, cu, padding_side="middle")


def test_compiled_fullgraph():
    import fma_b200

    lens = [0, 70, 170, 295]
    cu = torch.tensor(lens, dtype=torch.uint32, device=DEV)
    x = randn((3, 128, 24), torch.bfloat16, 1).to(DEV)
    fn = torch.compile(fma_b200.pack_sequence, fullgraph=True)
    got = fn(x, cu_seqlens=cu, output_shape=(295, 24), padding_side="left")
    np.testing.assert_array_equal(to_np(got), O.pack_sequence(to_np(x), np.array(lens), "left"))
    fn2 = torch.compile(fma_b200.unpack_sequence, fullgraph=True)
    got2 = fn2(got, cu_seqlens=cu, output_shape=(3, 128, 24), padding_side="left")
    np.testing.assert_array_equal(to_np(got2), O.unpack_sequence(to_np(got), np.array(lens), (3, 128, 24), "left"))
