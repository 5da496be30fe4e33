"""Matrix products and triangle masks (minit/functional/linalg.py:9-45).

``matrix_multiply(x, y)``: y is the [N, K] weight of a linear layer (minit/cuda/dispatch.py:59-78) or a
``QuantizedTensor``, whose product goes through this package's dispatch table to the fused GPTQ kernels
(the quantized rule of minit/quantize/dispatch.py:8-11) -- that path needs the CUDA library and a GPU."""
from __future__ import annotations

import torch

from .shape import expand, fold
from .utils import integer, unwrap, wrap

__all__ = ["matrix_multiply", "batch_matrix_multiply", "triangle_upper", "triangle_lower"]


def matrix_multiply(x, y):
    from ...quantize.tensor import QuantizedTensor
    from ..collective import CollectiveTensor, matrix_multiply as placed
    from ...collective.quantized import ShardedQuantized
    if isinstance(x, CollectiveTensor) or isinstance(y, (CollectiveTensor, ShardedQuantized)):
        return placed(x, y, matrix_multiply)
    if isinstance(x, torch.Tensor):                             # torch operands: the package's own torch-level function
        from ...functional.linalg import matrix_multiply as on_torch
        return on_torch(x, y)
    assert len(y.shape) == 2
    ms = None
    if len(x._shape) > 2:
        ms = x._shape[:-1]
        x = fold(x, 0, len(ms))
    if isinstance(y, QuantizedTensor):
        from ...functional.linalg import matrix_multiply as fused
        z = wrap(fused(unwrap(x), y))
    else:
        assert x.dtype == y.dtype
        z = wrap(torch.matmul(unwrap(x), unwrap(y).t()))
    return z if ms is None else expand(z, 0, ms)


def batch_matrix_multiply(x, y):
    """[..., M, K] x [..., N, K] -> [..., M, N]"""
    assert len(x._shape) > 2 and len(y._shape) > 2
    return wrap(torch.matmul(unwrap(x), unwrap(y).transpose(-1, -2)))


def _triangle(x, diagonal, upper: bool):
    t = unwrap(x)
    rows = torch.arange(t.shape[-2], device=t.device)[:, None]
    cols = torch.arange(t.shape[-1], device=t.device)[None, :]
    d = integer(diagonal)
    keep = (rows + d <= cols) if upper else (rows > cols + d)
    return wrap(torch.where(keep, t, torch.zeros((), dtype=t.dtype, device=t.device)))


def triangle_upper(x, diagonal):
    """keeps x[..., i, j] where i + diagonal <= j, zero elsewhere (minit/cuda/dispatch.py:384-404)"""
    return _triangle(x, diagonal, True)


def triangle_lower(x, diagonal):
    """keeps x[..., i, j] where i > j + diagonal, zero elsewhere (minit/cuda/dispatch.py:407-427)"""
    return _triangle(x, diagonal, False)
