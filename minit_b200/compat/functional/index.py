"""Slicing, gathering and concatenation (minit/functional/index.py:8-50; device rules: minit/cuda/dispatch.py:271-352)."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from .utils import integer, integers, unwrap, wrap

__all__ = ["slice", "slice_set", "index", "index_set", "split", "tie"]


def slice(x, start, stop, axis: int):
    start, stop = integer(start), integer(stop)
    assert 0 <= start <= stop <= x._shape[axis]
    return wrap(unwrap(x).narrow(axis, start, stop - start))


def slice_set(x, start, stop, axis: int, value):
    """a copy of x with [start, stop) of the axis replaced"""
    start, stop = integer(start), integer(stop)
    z = unwrap(x).clone()
    z.narrow(axis, start, stop - start).copy_(unwrap(value))
    return wrap(z)


def index(x, index, axis: int):
    """gather whole slices of the axis by a 1-D int32 index"""
    assert index.dtype == "int32" and len(index._shape) == 1
    return wrap(unwrap(x).index_select(axis, unwrap(index).long()))


def index_set(x, index, axis: int, value):
    z = unwrap(x).clone()
    z.index_copy_(axis, unwrap(index).long(), unwrap(value))
    return wrap(z)


def split(x, axis: int, sizes: Sequence) -> Tuple:
    sizes = integers(sizes)
    assert sum(sizes) == x._shape[axis]
    parts, offset = [], 0
    for size in sizes:
        parts.append(slice(x, offset, offset + size, axis))
        offset += size
    return tuple(parts)


def tie(xs: Sequence, axis: int):
    """concatenation along the axis"""
    return wrap(torch.cat([unwrap(x) for x in xs], dim=axis))
