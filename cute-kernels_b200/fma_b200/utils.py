"""Small host helpers with the reference's names (fma/utils/contiguous.py:15-21, fma/utils/random.py:11-16)."""

from __future__ import annotations

import functools
import random
from typing import Any, Callable

import numpy as np
import torch
from torch.utils._pytree import tree_map


def _make_contiguous(x: Any) -> Any:
    return x.contiguous() if isinstance(x, torch.Tensor) else x


def ensure_contiguous(func: Callable) -> Callable:
    """Decorator: every tensor argument is made contiguous before the call."""

    @functools.wraps(func)
    def inner(*args, **kwargs):
        return func(*tree_map(_make_contiguous, args), **tree_map(_make_contiguous, kwargs))

    return inner


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def ceil_divide(x: int, y: int) -> int:
    return (x + y - 1) // y
