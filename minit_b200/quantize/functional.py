"""``dequantize(x, group, zero, scale, axis)`` (reference: minit/quantize/functional.py:6-8)."""
from ..core.dispatch import dispatch
from .operator import Dequantize


def dequantize(x, group, zero, scale, axis: int):
    (z,) = dispatch(Dequantize(axis), x, group, zero, scale)
    return z
