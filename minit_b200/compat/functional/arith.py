"""Elementwise arithmetic with the reference's names and operand rules (minit/functional/arith.py:9-157): a Python
number next to a tensor becomes a constant of the tensor's dtype; two host scalars are combined on the host; a device
tensor and a one-element operand broadcast.  Integer division truncates, as the generated C expression ``a / b`` does
(minit/cuda/dispatch.py:134-147)."""
from __future__ import annotations

import math
import operator
from numbers import Number
from typing import Optional

import torch

from ..tensor import CUDATensor, ScalarTensor, Tensor, python_type, torch_dtype
from .utils import is_device, number, scalar_dtype, unwrap, wrap

__all__ = ["add", "subtract", "multiply", "divide", "floor_divide", "modulo", "power", "exponential", "logarithm", "square",
           "square_root", "sine", "cosine", "constant", "cast", "greater_than", "equal", "not_equal", "less_than", "logical_and",
           "logical_not", "logical_or", "greater_equal", "less_equal", "select_max", "select", "where"]


def _operands(*args):
    """torch operands of an elementwise rule: host scalars become 0-d tensors of the device operands' dtype."""
    lead = next(arg for arg in args if is_device(arg))
    t = unwrap(lead)
    out = []
    for arg in args:
        if is_device(arg):
            assert arg.dtype == lead.dtype, f"{arg.dtype} vs {lead.dtype}"
            out.append(unwrap(arg))
        else:
            out.append(torch.tensor(number(arg), dtype=t.dtype, device=t.device))
    return out


def _host(fn, *args, dtype: Optional[str] = None) -> ScalarTensor:
    dtype = dtype or scalar_dtype(*args)
    value = fn(*[number(arg) for arg in args])
    return ScalarTensor(python_type(dtype)(value), (), dtype)


def _elementwise(device_fn, host_fn, *args, result_dtype: Optional[str] = None):
    if any(is_device(arg) for arg in args):
        return wrap(device_fn(*_operands(*args)))
    return _host(host_fn, *args, dtype=result_dtype)


def _divide(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return torch.div(x, y) if x.dtype.is_floating_point else torch.div(x, y, rounding_mode="trunc")


def _host_divide(x, y):
    return x / y if isinstance(x, float) or isinstance(y, float) else int(x / y)


def add(x, y):
    return _elementwise(torch.add, operator.add, x, y)


def subtract(x, y):
    return _elementwise(torch.sub, operator.sub, x, y)


def multiply(x, y):
    return _elementwise(torch.mul, operator.mul, x, y)


def divide(x, y):
    return _elementwise(_divide, _host_divide, x, y)


def floor_divide(x, y):
    return _elementwise(lambda a, b: torch.div(a, b, rounding_mode="floor"), operator.floordiv, x, y)


def modulo(x, y):
    return _elementwise(torch.remainder, operator.mod, x, y)


def power(base, exponent):
    return _elementwise(torch.pow, pow, base, exponent)


def exponential(x):
    return _elementwise(torch.exp, math.exp, x)


def logarithm(x):
    return _elementwise(torch.log, math.log, x)


def square(x):
    return multiply(x, x)


def square_root(x):
    return _elementwise(torch.sqrt, math.sqrt, x)


def sine(x):
    return _elementwise(torch.sin, math.sin, x)


def cosine(x):
    return _elementwise(torch.cos, math.cos, x)


def constant(x: Number, dtype: str) -> ScalarTensor:
    assert not isinstance(x, Tensor)
    return ScalarTensor(x, (), dtype)


def cast(x, dtype: str):
    if x.dtype == dtype:
        return x
    if is_device(x):
        return wrap(unwrap(x).to(torch_dtype(dtype)))
    return ScalarTensor(python_type(dtype)(number(x)), (), dtype)


def greater_than(x, y):
    return _elementwise(torch.gt, operator.gt, x, y, result_dtype="bool")


def equal(x, y):
    return _elementwise(torch.eq, operator.eq, x, y, result_dtype="bool")


def not_equal(x, y):
    return _elementwise(torch.ne, operator.ne, x, y, result_dtype="bool")


def less_than(x, y):
    return _elementwise(torch.lt, operator.lt, x, y, result_dtype="bool")


def greater_equal(x, y):
    return _elementwise(torch.ge, operator.ge, x, y, result_dtype="bool")


def less_equal(x, y):
    return _elementwise(torch.le, operator.le, x, y, result_dtype="bool")


def logical_and(x, y):
    return _elementwise(torch.logical_and, lambda a, b: bool(a) and bool(b), x, y, result_dtype="bool")


def logical_or(x, y):
    return _elementwise(torch.logical_or, lambda a, b: bool(a) or bool(b), x, y, result_dtype="bool")


def logical_not(x):
    return _elementwise(torch.logical_not, lambda a: not a, x, result_dtype="bool")


def select_max(x, y):
    return _elementwise(torch.maximum, max, x, y)


def select(index, *args, dtype: Optional[str] = None):
    """``args[index]`` elementwise (minit/functional/arith.py:145-148)."""
    assert is_device(index), "select takes a device index"
    idx = unwrap(index).long()
    values = [arg for arg in args if is_device(arg)]
    target = torch_dtype(dtype or (values[0].dtype if values else scalar_dtype(*args)))
    out = torch.empty(idx.shape, dtype=target, device=idx.device)
    for i, arg in enumerate(args):
        src = unwrap(arg).to(target).expand(idx.shape) if is_device(arg) else torch.full(idx.shape, number(arg), dtype=target, device=idx.device)
        out = torch.where(idx == i, src, out)
    return wrap(out)


def where(condition, true_value, false_value, *, dtype: Optional[str] = None):
    assert condition.dtype == "bool"
    return select(condition, false_value, true_value, dtype=dtype)
