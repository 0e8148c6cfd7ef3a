"""continuous_count on the GPU (through the C ABI) against torch.bincount, the CPU oracle and the
reference-generated golden counts.  Bit-exact."""

import numpy as np
import pytest
import torch

from _util import DEV, to_np, zipf_ids

pytestmark = pytest.mark.gpu


def _count(ids, size, variant=None):
    from fma_b200 import continuous_count

    out = continuous_count(ids, size, _variant=variant)
    assert out.dtype == torch.uint32 and out.shape == (size,)
    return to_np(out)


def test_golden_cases(golden_dir):
    z = np.load(golden_dir / "continuous_count.npz")
    for i in range(int(z["n_cases"])):
        ids, size, ref = z[f"ids_{i}"], int(z[f"size_{i}"]), z[f"count_{i}"]
        for variant in (None, 0, 1, 2):
            if variant == 2 and size > 1024:
                continue
            got = _count(torch.from_numpy(ids).to(DEV), size, variant)
            np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("variant", [None, 0, 1, 2])
def test_sizes_like_the_reference_suite(dtype, variant):
    # sizes 2^i + j as in tests/ops/continuous_count_test.py of the reference (72 bins), thinned
    g = torch.Generator().manual_seed(7)
    for i in range(0, 15, 2):
        for j in (0, 1, 3, 9):
            n = 2**i + j
            ids = torch.randint(0, 72, (n,), generator=g).to(dtype)
            got = _count(ids.to(DEV), 72, variant)
            np.testing.assert_array_equal(got, torch.bincount(ids.long(), minlength=72).numpy())


@pytest.mark.parametrize("dist", ["uniform", "zipf"])
@pytest.mark.parametrize("variant", [None, 0, 1, 2])
def test_full_size_16m_ids_128_bins(dist, variant):
    from oracle import int_oracle

    n, E = 2**24, 128
    if dist == "uniform":
        ids = torch.randint(0, E, (n,), dtype=torch.int32, generator=torch.Generator().manual_seed(0))
    else:
        ids = zipf_ids(n, E, 1.1, seed=1)
    got = _count(ids.to(DEV), E, variant)
    np.testing.assert_array_equal(got, torch.bincount(ids.long(), minlength=E).numpy())
    np.testing.assert_array_equal(got, int_oracle.count(ids.numpy(), E).astype(np.int64))
    assert got.sum() == n
    # a second call reuses the workspace (its ticket must have been reset)
    np.testing.assert_array_equal(_count(ids.to(DEV), E, variant), got)


def test_out_of_range_and_edge_cases():
    ids = torch.tensor([0, 5, -1, 3, 7, 3, 100, 2**31 - 1], dtype=torch.int32, device=DEV)
    np.testing.assert_array_equal(_count(ids, 4), [1, 0, 0, 2])
    ids64 = torch.tensor([0, 5, -1, 3, 2**40, 3], dtype=torch.int64, device=DEV)
    np.testing.assert_array_equal(_count(ids64, 4), [1, 0, 0, 2])
    np.testing.assert_array_equal(_count(torch.empty(0, dtype=torch.int32, device=DEV), 16), np.zeros(16))
    np.testing.assert_array_equal(_count(torch.zeros(77, dtype=torch.int64, device=DEV), 1), [77])
    big = torch.randint(0, 16384, (100003,), generator=torch.Generator().manual_seed(3))
    np.testing.assert_array_equal(_count(big.to(DEV), 16384), torch.bincount(big, minlength=16384).numpy())
    for size in (2, 3, 511, 512, 513, 1024):  # around the limit of the atomic-free scheme
        ids = torch.randint(-2, size + 2, (70001,), generator=torch.Generator().manual_seed(size))
        want = torch.bincount(ids[(ids >= 0) & (ids < size)], minlength=size).numpy()
        np.testing.assert_array_equal(_count(ids.to(DEV), size), want)
        np.testing.assert_array_equal(_count(ids.int().to(DEV), size), want)
    # a view that does not start on a 16-byte boundary, and a strided one
    odd = torch.randint(0, 9, (1001,), dtype=torch.int32, generator=torch.Generator().manual_seed(4))
    np.testing.assert_array_equal(_count(odd.to(DEV)[1:], 9), torch.bincount(odd[1:].long(), minlength=9).numpy())
    np.testing.assert_array_equal(_count(odd.to(DEV)[::3], 9), torch.bincount(odd[::3].long(), minlength=9).numpy())

