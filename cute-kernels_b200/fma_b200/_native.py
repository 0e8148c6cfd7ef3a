"""ctypes binding of libfma_b200.so, the C-ABI library of sm_100a kernels.

There is no CPU or PyTorch fallback: if the library is missing, or a call returns a non-zero
status, a RuntimeError is raised.  `include/fma_b200.h` is the authoritative declaration of every
entry point; the argument types below mirror it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_int32, c_int64, c_void_p
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libfma_b200.so"

F32 = 0
BF16 = 1
F16 = 2

_I32, _I64, _P = c_int32, c_int64, c_void_p

# name -> (restype, argtypes); keep in the order of include/fma_b200.h
SIGNATURES: dict[str, tuple] = {
    "fma_b200_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "fma_b200_last_error": (ctypes.c_char_p, []),
    "fma_b200_abi_version": (ctypes.c_int, []),
    "fma_b200_set_sm_limit": (ctypes.c_int, [_I32]),
    "fma_b200_device_status": (ctypes.c_int, [_P, _P]),
    "fma_b200_device_status_peek": (ctypes.c_int, [_P, _P]),
    "fma_b200_continuous_count_workspace_bytes": (_I64, [_I32]),
    "fma_b200_continuous_count": (ctypes.c_int, [_P, _I32, _I64, _I32, _P, _P, _I64, _P]),
    "fma_b200_continuous_count_variant": (ctypes.c_int, [_P, _I32, _I64, _I32, _P, _P, _I64, _I32, _P]),
    "fma_b200_continuous_count_static": (ctypes.c_int, [_P, _I32, _I64, _I32, _P, _P]),
    "fma_b200_router_topk_softmax": (ctypes.c_int, [_P, _I32, _I64, _I32, _I32, _P, _P, _P]),
    "fma_b200_router_topk_softmax_routed": (ctypes.c_int, [_P, _I32, _I64, _I32, _I32, _P, _P, _I32, _P, _I64, _P]),
    "fma_b200_router_topk_softmax_backward": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _P, _P]),
    "fma_b200_router_mean_prob_backward": (ctypes.c_int, [_P, _P, _I32, _I64, _I32, _P, _P]),
    "fma_b200_moe_rows_cap": (_I64, [_I64, _I32, _I32]),
    "fma_b200_moe_sort_workspace_bytes": (_I64, [_I64, _I32]),
    "fma_b200_moe_sort": (ctypes.c_int, [_P, _I64, _I32, _I32, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _P]),
    "fma_b200_moe_sort_routed": (
        ctypes.c_int,
        [_P, _I64, _I32, _I32, _I32, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _P],
    ),
    "fma_b200_moe_ep_recv_maps": (ctypes.c_int, [_P, _I32, _I32, _I32, _I64, _P, _P, _P]),
    "fma_b200_moe_scatter": (ctypes.c_int, [_P, _I32, _I64, _I32, _I32, _P, _P, _P, _I32, _I64, _P, _P]),
    "fma_b200_moe_scatter_backward": (ctypes.c_int, [_P, _I32, _I64, _I32, _I32, _P, _P, _P]),
    "fma_b200_moe_combine": (ctypes.c_int, [_P, _P, _I32, _I64, _I32, _I32, _P, _P, _P]),
    "fma_b200_moe_combine_backward": (
        ctypes.c_int,
        [_P, _P, _P, _I32, _I64, _I32, _I32, _P, _P, _P, _I32, _I64, _P, _P, _P],
    ),
    "fma_b200_moe_bias_add": (ctypes.c_int, [_P, _P, _I32, _I64, _I32, _P, _P, _P]),
    "fma_b200_moe_bias_grad": (ctypes.c_int, [_P, _I32, _I32, _I32, _P, _P, _P]),
    "fma_b200_moe_zero_padding": (ctypes.c_int, [_P, _I64, _P, _P, _I32, _P]),
    "fma_b200_moe_gemm_forward_peer": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_moe_gemm_dgrad_peer": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_peer_buffer_create": (ctypes.c_int, [_I64, _P, _P]),
    "fma_b200_peer_buffer_open": (ctypes.c_int, [_P, _P]),
    "fma_b200_peer_buffer_close": (ctypes.c_int, [_P]),
    "fma_b200_peer_buffer_destroy": (ctypes.c_int, [_P]),
    "fma_b200_peer_copy": (ctypes.c_int, [_I32, _P, _P, _P, _P]),
    "fma_b200_peer_signal": (ctypes.c_int, [_I32, _P, _I32, _P]),
    "fma_b200_peer_wait": (ctypes.c_int, [_P, _I32, _I32, _I32, _P]),
    "fma_b200_swiglu_forward": (ctypes.c_int, [_P, _I64, _P, _I64, _P, _I64, _I32, _I64, _I64, _P]),
    "fma_b200_swiglu_backward": (
        ctypes.c_int,
        [_P, _I64, _P, _I64, _P, _I64, _P, _I64, _P, _I64, _I32, _I64, _I64, _P],
    ),
    "fma_b200_pack_sequence": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I32, _P]),
    "fma_b200_unpack_sequence": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I32, _P]),
    "fma_b200_moe_gemm_forward": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_moe_gemm_dgrad": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_moe_gemm_wgrad": (ctypes.c_int, [_P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_moe_gemm_forward_swiglu": (ctypes.c_int, [_P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_moe_gemm_dgrad_swiglu": (ctypes.c_int, [_P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _I32, _P]),
    "fma_b200_grouped_gemm_workspace_bytes": (_I64, [_I32, _I64]),
    "fma_b200_grouped_gemm": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _P, _I64, _P]),
}

_lib: ctypes.CDLL | None = None


def library_path() -> Path:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build the CUDA kernels with `python cute-kernels_b200/build.py` "
                "(there is no CPU fallback)"
            )
        handle = ctypes.CDLL(os.fspath(_LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means header and library disagree
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


# Kernels launched per entry-point call (the sort is three kernels; status queries launch none).
KERNELS_PER_CALL = {
    "fma_b200_moe_sort": 3, "fma_b200_moe_sort_routed": 2, "fma_b200_device_status": 0, "fma_b200_device_status_peek": 0, "fma_b200_set_sm_limit": 0, "fma_b200_peer_buffer_create": 0,
    "fma_b200_peer_buffer_open": 0, "fma_b200_peer_buffer_close": 0, "fma_b200_peer_buffer_destroy": 0,
    "fma_b200_peer_copy": 0,
    "fma_b200_moe_gemm_wgrad": 2,  # expert order + GEMM for the 16-bit types (one kernel for fp32)
}  # fmt: skip
launch_count = 0  # kernels launched through this binding since import (a plain counter for benchmarks)
_timing: dict[str, list] | None = None  # entry point -> [(start event, end event)], when enabled


def enable_timing(enabled: bool) -> None:
    """Benchmark hook: bracket every entry-point call with CUDA events on the launching stream."""
    global _timing
    _timing = {} if enabled else None


def collect_timing() -> dict[str, tuple[int, float]]:
    """Returns {entry point: (calls, total milliseconds)} and clears the record.  Synchronises."""
    global _timing
    out: dict[str, tuple[int, float]] = {}
    if _timing is None:
        return out
    torch.cuda.synchronize()
    for name, pairs in _timing.items():
        out[name] = (len(pairs), sum(a.elapsed_time(b) for a, b in pairs))
    _timing = {}
    return out


def call(name: str, *args) -> None:
    """Calls an int-status entry point and raises RuntimeError on a non-zero status."""
    global launch_count
    handle = lib()
    launch_count += KERNELS_PER_CALL.get(name, 1)
    if _timing is not None and KERNELS_PER_CALL.get(name, 1) > 0:
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        status = getattr(handle, name)(*args)
        end.record()
        _timing.setdefault(name, []).append((start, end))
    else:
        status = getattr(handle, name)(*args)
    if status != 0:
        text = handle.fma_b200_status_string(status).decode()
        detail = handle.fma_b200_last_error().decode()
        raise RuntimeError(f"{name} failed: {text} ({detail})")


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(None) if t is None else c_void_p(t.data_ptr())


def stream_ptr(device: torch.device | None = None) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return F16
    raise RuntimeError(f"unsupported dtype {dtype}: the B200 kernels handle float32, bfloat16 and float16")


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("this op runs on CUDA tensors only (no CPU fallback exists)")


def device_status(device: torch.device | None = None) -> int:
    """Reads and clears the device status word (0 = no kernel reported an error); synchronises."""
    out = c_int32(0)
    call("fma_b200_device_status", ctypes.cast(ctypes.pointer(out), c_void_p), stream_ptr(device))
    return out.value
