"""``matrix_multiply(x, y)``: folds the leading dims of x to M, dispatches MatrixMultiply and
unfolds (reference: minit/functional/linalg.py:9-20)."""
from __future__ import annotations

from ..core.dispatch import dispatch
from ..operator.linalg import MatrixMultiply


def matrix_multiply(x, y):
    assert len(y.shape) == 2
    ms = None
    if x.dim() > 2:
        ms = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
    (z,) = dispatch(MatrixMultiply(), x, y)
    if ms is not None:
        z = z.reshape(*ms, z.shape[-1])
    return z
