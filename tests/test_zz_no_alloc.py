"""fma_b200_continuous_count_static: the histogram for callers that cannot allocate device memory.

Some users of the library (a plugin inside a host that owns the GPU memory pool, code that must not
trigger cudaMalloc's device-wide synchronisation, a bare C program) cannot hand the kernel a scratch
buffer, so this entry point keeps its scratch in an array that is part of the library image.  The
test calls it through the C ABI exactly as such a caller would: it passes only the ids and the output
array.  The result must equal, bit for bit, what the workspace-based entry point returns, on two
calls in a row (the second call reuses the scratch the first one left behind).

Collected last on purpose (file name), so that a run that stops at the first failure has already
run every other test; it must also pass alone in a fresh process.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(ids: torch.Tensor, size: int):
    from fma_b200 import _native

    lib = _native.lib()
    stream = _native.stream_ptr(ids.device)
    out_static = torch.full((size,), 0xDEAD, dtype=torch.int32, device=ids.device)  # garbage to overwrite
    out_ws = torch.empty(size, dtype=torch.int32, device=ids.device)
    nbytes = lib.fma_b200_continuous_count_workspace_bytes(size)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=ids.device)
    _native.call("fma_b200_continuous_count_static", _native.ptr(ids), ids.element_size(), ids.numel(), size,
                 _native.ptr(out_static), stream)
    _native.call("fma_b200_continuous_count", _native.ptr(ids), ids.element_size(), ids.numel(), size,
                 _native.ptr(out_ws), _native.ptr(ws), nbytes, stream)
    torch.cuda.synchronize()
    return out_static.cpu(), out_ws.cpu()


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(dtype):
    g = torch.Generator().manual_seed(11)
    first = torch.randint(0, 128, (1 << 22,), generator=g).to(dtype)
    second = torch.randint(0, 1000, (777_777,), generator=g).to(dtype)  # other size, other grid, same scratch
    for ids, size in ((first, 128), (second, 1000), (first, 128)):
        a, b = _both(ids.cuda(), size)
        assert torch.equal(a, b)
        assert torch.equal(a.long(), torch.bincount(ids.long(), minlength=size))


def test_static_scratch_edge_cases_and_limit():
    from fma_b200 import _native

    lib = _native.lib()
    a, b = _both(torch.empty(0, dtype=torch.int32, device="cuda"), 16)
    assert torch.equal(a, b) and int(a.sum()) == 0
    ids = torch.tensor([3, -1, 3, 99, 0], dtype=torch.int32, device="cuda")
    a, b = _both(ids, 4)
    assert a.tolist() == [1, 0, 0, 2] == b.tolist()
    # beyond the built-in scratch: refused with a clear message, nothing launched
    out = torch.zeros(2048, dtype=torch.int32, device="cuda")
    rc = lib.fma_b200_continuous_count_static(_native.ptr(ids), 4, ids.numel(), 2048, _native.ptr(out),
                                              ctypes.c_void_p(None))
    assert rc == 1
    assert b"1024" in lib.fma_b200_last_error()
    with pytest.raises(RuntimeError, match="exceeds"):
        _native.call("fma_b200_continuous_count_static", _native.ptr(ids), 4, ids.numel(), 1025, _native.ptr(out),
                     ctypes.c_void_p(None))
