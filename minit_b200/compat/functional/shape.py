"""Shape operators (minit/functional/shape.py:11-73; device rules: minit/cuda/dispatch.py:209-268, 355-381, 481-490).
``add_axis``, ``remove_axis``, ``fold``, ``expand`` and ``reinterpret`` are views of the same memory, as in the
reference; ``broadcast`` and ``transpose`` make a new tensor."""
from __future__ import annotations

from typing import Optional, Sequence

from ..tensor import CUDATensor, ScalarTensor, dtype_size
from .utils import integer, integers, is_device, unwrap, wrap

__all__ = ["fold", "expand", "add_axis", "remove_axis", "broadcast", "transpose", "repeat", "repeat_interleaved", "reinterpret"]


def _view(x: CUDATensor, shape) -> CUDATensor:
    return CUDATensor.wrap(tuple(shape), x.dtype, x.memory)


def fold(x, start: int, stop: int):
    """axes [start, stop) become one"""
    if stop - start == 1:
        return x
    size = 1
    for dim in x._shape[start:stop]:
        size *= dim
    return _view(x, x._shape[:start] + (size,) + x._shape[stop:])


def expand(x, axis: int, sizes: Sequence):
    """axis becomes len(sizes) axes whose product is its length"""
    if len(sizes) == 1:
        return x
    sizes = integers(sizes)
    size = 1
    for dim in sizes:
        size *= dim
    assert size == x._shape[axis], f"expand {x._shape[axis]} into {sizes}"
    return _view(x, x._shape[:axis] + sizes + x._shape[axis + 1:])


def add_axis(x, axis: int, size=None):
    if not is_device(x):                                      # a host scalar grows a unit axis (minit/functional/shape.py:68-73)
        assert size is None
        return ScalarTensor(x.value(), x.shape[:axis] + (ScalarTensor(1, (), "int32"),) + x.shape[axis:], x.dtype)
    z = _view(x, x._shape[:axis] + (1,) + x._shape[axis:])
    return z if size is None else broadcast(z, axis, size)


def remove_axis(x, axis: int):
    assert x._shape[axis] == 1
    return _view(x, x._shape[:axis] + x._shape[axis + 1:])


def broadcast(x, axis: int, size):
    assert axis < len(x._shape) and x._shape[axis] == 1
    shape = list(x._shape)
    shape[axis] = integer(size)
    return wrap(unwrap(x).expand(shape))


def transpose(x, axis_a: int, axis_b: int):
    if axis_a == axis_b:
        return x
    return wrap(unwrap(x).transpose(axis_a, axis_b))


def repeat(x, axis: int, size):
    """the whole axis ``size`` times over"""
    return fold(broadcast(add_axis(x, axis), axis, size), axis, axis + 2)


def repeat_interleaved(x, axis: int, size):
    """every element of the axis ``size`` times in a row"""
    return fold(broadcast(add_axis(x, axis + 1), axis + 1, size), axis, axis + 2)


def reinterpret(x, target: str):
    """the same bytes as another dtype; the last axis absorbs the size ratio"""
    source_size, target_size = dtype_size(x.dtype), dtype_size(target)
    last = x._shape[-1]
    new_last = last * source_size // target_size
    assert new_last * target_size // source_size == last
    return CUDATensor.wrap(x._shape[:-1] + (new_last,), target, x.memory)
