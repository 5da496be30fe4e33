"""Tensor-parallel rules for MatrixMultiply (reference: minit/collective/dispatch.py:26-44).

Dense weights are [N,K]: Split(0) is column-parallel (output Split(1)), Split(1) is
row-parallel (x sliced on K, output Partial), Broadcast is replicated.  A sharded quantized
weight (``ShardedQuantized``) states its parallel mode directly because its packed layout is
[K/pack, N]."""
from __future__ import annotations

import torch

from ..core.dispatch import register_dispatch
from ..functional.linalg import matrix_multiply
from ..operator.linalg import MatrixMultiply
from .quantized import ShardedQuantized
from .spec import CollectiveSpecBroadcast, CollectiveSpecSplit
from .tensor import CollectiveTensor


def _both_collective(x, y):
    return isinstance(x, CollectiveTensor) and isinstance(y, CollectiveTensor)


@register_dispatch(MatrixMultiply, predicate=_both_collective, priority=2)
def dispatch_collective_matmul(op: MatrixMultiply, x: CollectiveTensor, y: CollectiveTensor):
    communicator = x._communicator
    spec = y.spec
    if isinstance(spec, CollectiveSpecSplit) and spec.axis == 0:
        x = x.to_broadcast()
        return (CollectiveTensor.from_split(communicator, matrix_multiply(x._local, y._local), x.dim() - 1),)
    if isinstance(spec, CollectiveSpecSplit) and spec.axis == 1:
        x = x.to_split(x.dim() - 1)
        return (CollectiveTensor.from_partial(communicator, matrix_multiply(x._local, y._local)),)
    if isinstance(spec, CollectiveSpecBroadcast):
        x = x.to_broadcast()
        return (CollectiveTensor.from_broadcast(communicator, matrix_multiply(x._local, y._local)),)
    raise TypeError(f"no tensor-parallel matmul rule for a weight placed as {spec}")


def _x_collective_w_sharded(x, y):
    return isinstance(x, CollectiveTensor) and isinstance(y, ShardedQuantized)


@register_dispatch(MatrixMultiply, predicate=_x_collective_w_sharded, priority=3)
def dispatch_collective_quantized_matmul(op: MatrixMultiply, x: CollectiveTensor, y: ShardedQuantized):
    communicator = x._communicator
    if y.mode == "column":
        x = x.to_broadcast()
        return (CollectiveTensor.from_split(communicator, y.local_matmul(x._local), x.dim() - 1),)
    x = x.to_split(x.dim() - 1)
    return (CollectiveTensor.from_partial(communicator, y.local_matmul(x._local)),)
