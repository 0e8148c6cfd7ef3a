"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import numpy as np
import torch

DEV = "cuda"

# rel-L2 bars from the benchmark specification: bf16 <= 1e-2, fp32 <= 1e-5
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}
ORACLE_DTYPE = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    if t.dtype == torch.uint32:
        t = t.to(torch.int64)
    return t.cpu().numpy()


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))


def randn(shape, dtype, seed, scale=1.0) -> torch.Tensor:
    """Seeded N(0, scale) values generated on the CPU (so every device sees the same bits)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def zipf_ids(n: int, E: int, s: float, seed: int, dtype=torch.int32) -> torch.Tensor:
    """ids with P(rank r) ~ r^-s over a seeded random permutation of the E values."""
    p = 1.0 / np.arange(1, E + 1, dtype=np.float64) ** s
    cdf = np.cumsum(p / p.sum())
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(E, generator=g)
    u = torch.rand(n, dtype=torch.float64, generator=g)
    rank = torch.searchsorted(torch.from_numpy(cdf), u).clamp_(max=E - 1)
    return perm[rank].to(dtype)


def check_device_status():
    from fma_b200 import _native

    assert _native.device_status() == 0, "a kernel recorded a device-side error (bounded wait ran out)"
