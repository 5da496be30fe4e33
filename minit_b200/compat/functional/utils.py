"""Shared helpers of the functional layer: telling host scalars from device tensors and moving between the wrapper
types and torch."""
from __future__ import annotations

from numbers import Number
from typing import Sequence, Tuple

import torch

from ..tensor import CUDATensor, MetaTensor, ScalarTensor, Tensor, as_torch, dtype_name, torch_dtype


def is_device(x) -> bool:
    return isinstance(x, CUDATensor)


def number(x):
    """Python number of a host scalar (or of a one-element device tensor)."""
    if isinstance(x, ScalarTensor):
        return x.value()
    if isinstance(x, CUDATensor):
        assert len(x._shape) == 0
        return x.item()
    assert isinstance(x, Number), f"number expected, got {type(x).__name__}"
    return x


def integer(x) -> int:
    return int(number(x))


def integers(xs: Sequence) -> Tuple[int, ...]:
    return tuple(integer(x) for x in xs)


def wrap(t: torch.Tensor) -> CUDATensor:
    return CUDATensor.from_torch(t)


def unwrap(x) -> torch.Tensor:
    assert not isinstance(x, MetaTensor), "a buffer that was never loaded reached an operator"
    assert isinstance(x, CUDATensor), f"device tensor expected, got {type(x).__name__}"
    return as_torch(x)


def scalar_dtype(*args, default=None) -> str:
    """dtype name of a result computed on the host: the first tensor argument decides, else the Python type."""
    for arg in args:
        if isinstance(arg, Tensor):
            return arg.dtype
    if default is not None:
        return default
    for arg in args:
        if isinstance(arg, float):
            return "float32"
    return "bool" if all(isinstance(arg, bool) for arg in args) else "int32"


__all__ = ["is_device", "number", "integer", "integers", "wrap", "unwrap", "scalar_dtype", "dtype_name", "torch_dtype"]
