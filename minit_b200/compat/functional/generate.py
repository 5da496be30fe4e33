"""Tensor generators (minit/functional/generate.py:9-29; kernels: minit/cuda/dispatch.py:176-207)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..tensor import Tensor, current_device, torch_dtype
from .utils import integer, integers, number, wrap

__all__ = ["generate_interval", "generate_sequence", "fill"]


def generate_sequence(start, size, step=1, *, dtype: str):
    """``start + i * step`` for i in [0, size)"""
    t = torch_dtype(dtype)
    work = torch.float32 if t in (torch.float16, torch.bfloat16) else t
    i = torch.arange(integer(size), dtype=work, device=current_device())
    return wrap((i * number(step) + number(start)).to(t))


def generate_interval(start, stop, step=1, *, dtype: str):
    return wrap(torch.arange(number(start), number(stop), number(step), dtype=torch_dtype(dtype), device=current_device()))


def fill(value, shape: Sequence, dtype: Optional[str] = None):
    if isinstance(value, Tensor):
        assert len(value.shape) == 0 and (dtype is None or dtype == value.dtype)
        dtype = value.dtype
    assert dtype is not None, "fill of a Python number needs a dtype"
    return wrap(torch.full(integers(shape), number(value), dtype=torch_dtype(dtype), device=current_device()))
