"""ctypes access to the C integer oracle (int_oracle.c).  TEST INFRASTRUCTURE ONLY."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = _DIR / "libint_oracle.so"
_handle = None


def build() -> Path:
    subprocess.run(["make", "-C", str(_DIR), "libint_oracle.so"], check=True, capture_output=True)
    return _LIB


def _lib():
    global _handle
    if _handle is None:
        if not _LIB.exists():
            build()
        _handle = ctypes.CDLL(str(_LIB))
    return _handle


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def count(ids: np.ndarray, size: int) -> np.ndarray:
    ids = np.ascontiguousarray(ids)
    assert ids.dtype in (np.int32, np.int64)
    out = np.empty(size, dtype=np.uint32)
    rc = _lib().oracle_count(_p(ids), ctypes.c_int(ids.itemsize), ctypes.c_int64(ids.size), ctypes.c_int32(size), _p(out))
    assert rc == 0
    return out


def sort_maps(selected: np.ndarray, E: int, row_align: int = 128) -> dict:
    flat = np.ascontiguousarray(selected, dtype=np.int64).reshape(-1)
    R = flat.size
    rows_cap = -(-(R + E * (row_align - 1)) // 128) * 128
    res = {
        "sorted_expert_idxs": np.empty(R, np.int64),
        "sorted_scattered_idxs": np.empty(R, np.int64),
        "expert_count": np.empty(E, np.uint32),
        "pad_offsets": np.empty(E + 1, np.int32),
        "row_of_slot": np.empty(R, np.int32),
        "slot_of_row": np.empty(rows_cap, np.int32),
        "mtile_expert": np.empty(rows_cap // 128, np.int32) if row_align % 128 == 0 else None,
    }
    rc = _lib().oracle_sort_maps(
        _p(flat), ctypes.c_int64(R), ctypes.c_int32(E), ctypes.c_int32(row_align), ctypes.c_int64(rows_cap),
        _p(res["sorted_expert_idxs"]), _p(res["sorted_scattered_idxs"]), _p(res["expert_count"]),
        _p(res["pad_offsets"]), _p(res["row_of_slot"]), _p(res["slot_of_row"]), _p(res["mtile_expert"]),
    )  # fmt: skip
    assert rc == 0, rc
    res["rows_cap"] = rows_cap
    return res
