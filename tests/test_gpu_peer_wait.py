"""The bounded device-side wait of the peer-memory transport, on one GPU and without any peer: a wait
on a flag that nobody sets runs into its time limit, records status 0x7002 and returns; while that
status stands, later waits return at once; after the host has read (and thereby cleared) the status,
signalling and waiting work normally.  Nothing here faults or hangs the GPU: the limit is 5 ms."""

import ctypes
import time

import pytest
import torch

from _util import DEV

pytestmark = pytest.mark.gpu


def _wait(flags: torch.Tensor, n: int, value: int, timeout_ms: int):
    from fma_b200 import _native

    _native.call("fma_b200_peer_wait", ctypes.c_void_p(flags.data_ptr()), n, value, timeout_ms,
                 _native.stream_ptr(flags.device))


def test_wait_that_runs_out_reports_and_later_waits_return_at_once():
    from fma_b200 import _native

    assert _native.device_status() == 0
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _wait(flags, 2, 1, 5)  # nobody signals: gives up after 5 ms
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    assert 0.004 <= first < 1.0, first
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    _wait(flags, 2, 1, 2000)  # would poll for 2 s, but the recorded timeout makes it return at once
    b.record()
    torch.cuda.synchronize()
    assert a.elapsed_time(b) < 100.0
    assert _native.device_status() == 0x7002
    assert _native.device_status() == 0  # the read cleared it

    # a normal exchange on the same flags: signal value 1 into flags 0 and 1, then wait for them
    addrs = (ctypes.c_uint64 * 2)(flags.data_ptr(), flags.data_ptr() + 4)
    _native.call("fma_b200_peer_signal", 2, addrs, 1, _native.stream_ptr(flags.device))
    _wait(flags, 2, 1, 2000)
    torch.cuda.synchronize()
    assert flags[:2].tolist() == [1, 1]
    assert _native.device_status() == 0
