"""Reductions that keep the reduced axis with length one (minit/functional/reduce.py:8-24, minit/cuda/dispatch.py:152-170)."""
from __future__ import annotations

import torch

from .utils import unwrap, wrap

__all__ = ["sum", "mean", "max"]


def _accumulate(t: torch.Tensor) -> torch.Tensor:
    return t.float() if t.dtype in (torch.float16, torch.bfloat16) else t


def sum(x, axis: int):
    t = unwrap(x)
    return wrap(_accumulate(t).sum(dim=axis, keepdim=True).to(t.dtype))


def mean(x, axis: int):
    from .arith import divide
    return divide(sum(x, axis), x._shape[axis])


def max(x, axis: int):
    return wrap(unwrap(x).amax(dim=axis, keepdim=True))
