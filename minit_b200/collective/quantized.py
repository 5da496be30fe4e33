"""Tensor-parallel GPTQ linears: the reference's sharding rule (q/k/v/gate/up split on
out-features, o/down split on in-features: examples/llama3_70b.py:298-310;
minit/collective/dispatch.py:26-37) applied to packed GPTQ tensors, with one all-reduce of
the [M, hidden] partial after each row-parallel projection (Partial -> all_reduce,
minit/collective/tensor.py:72-73).

Column-parallel outputs stay sharded and feed the next row-parallel projection directly, so
a decoder layer needs two all-reduces and no all-gather.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..distributed.communicator import DistributedCommunicator
from ..distributed.group import get_world
from ..module import Module
from ..qlinear import quantized_matrix_multiply


def shard_gptq_column(qweight, qzeros, scales, bits: int, rank: int, size: int):
    """Slice N: qweight[:, N_r], qzeros[:, N_r/pack], scales[:, N_r]; g_idx is unchanged."""
    pack = 32 // bits
    n = qweight.shape[1]
    if n % (size * pack) != 0:
        raise ValueError(f"out-features {n} do not split over {size} ranks on a {pack}-column boundary")
    lo, hi = n // size * rank, n // size * (rank + 1)
    return (qweight[:, lo:hi].contiguous(), None if qzeros is None else qzeros[:, lo // pack:hi // pack].contiguous(),
            scales[:, lo:hi].contiguous())


def shard_gptq_row(qweight, qzeros, scales, bits: int, rank: int, size: int, g_idx=None):
    """Slice K on group boundaries: qweight[K_r/pack, :], qzeros/scales[G_r, :].  With an
    act-order g_idx the groups of a K slice are not contiguous, so every rank keeps the full
    scale/zero tables and only qweight and g_idx are sliced."""
    pack = 32 // bits
    kp, g = qweight.shape[0], scales.shape[0]
    if kp % size != 0:
        raise ValueError(f"in-features {kp * pack} do not split over {size} ranks")
    qw = qweight[kp // size * rank:kp // size * (rank + 1)].contiguous()
    if g_idx is not None:
        k = kp * pack
        return qw, qzeros, scales, g_idx[k // size * rank:k // size * (rank + 1)].contiguous()
    if g % size != 0:
        raise ValueError(f"{g} groups do not split over {size} ranks")
    sl = slice(g // size * rank, g // size * (rank + 1))
    return qw, None if qzeros is None else qzeros[sl].contiguous(), scales[sl].contiguous(), None


class ShardedQuantized:
    """A rank's shard of a GPTQ weight plus its parallel mode ("column" or "row")."""

    def __init__(self, mode: str, qweight, qzeros, scales, g_idx, bits: int, bias=None) -> None:
        assert mode in ("column", "row")
        self.mode, self.qweight, self.qzeros, self.scales, self.g_idx, self.bits, self.bias = \
            mode, qweight, qzeros, scales, g_idx, bits, bias

    @property
    def shape(self):
        return (self.qweight.shape[0] * (32 // self.bits), self.qweight.shape[1])

    def local_matmul(self, x, out=None, flags: int = 0):
        return quantized_matrix_multiply(x, self.qweight, self.qzeros, self.scales, self.g_idx, bits=self.bits,
                                         bias=self.bias, out=out, flags=flags)


class ColumnParallelQLinear(Module):
    """x replicated [*, K] -> local output [*, N / world]."""

    def __init__(self, qweight, qzeros, scales, g_idx, bits: int, bias=None, *, rank=None, size=None) -> None:
        super().__init__()
        world = get_world()
        rank = world.rank if rank is None else rank
        size = world.size if size is None else size
        qw, qz, s = shard_gptq_column(qweight, qzeros, scales, bits, rank, size)
        if bias is not None:
            n = qweight.shape[1]
            bias = bias[n // size * rank:n // size * (rank + 1)].contiguous()
        self.shard = ShardedQuantized("column", qw, qz, s, g_idx, bits, bias)

    def forward(self, x, out=None, flags: int = 0):
        return self.shard.local_matmul(x, out=out, flags=flags)


class RowParallelQLinear(Module):
    """x sharded on K [*, K / world] -> partial [*, N], summed over ranks in place on the
    current stream.  The bias is added by rank 0 only, so the sum counts it once."""

    def __init__(self, communicator: Optional[DistributedCommunicator], qweight, qzeros, scales, g_idx, bits: int,
                 bias=None, *, rank=None, size=None, fused=None) -> None:
        super().__init__()
        world = get_world()
        rank = world.rank if rank is None else rank
        size = world.size if size is None else size
        self.communicator = communicator
        self.size = size
        self.rank = rank
        self.fused = fused   # a collective.fused.FusedAllReduce: GEMM and all-reduce become one kernel
        qw, qz, s, gi = shard_gptq_row(qweight, qzeros, scales, bits, rank, size, g_idx)
        self.shard = ShardedQuantized("row", qw, qz, s, gi, bits, bias if rank == 0 else None)

    def forward(self, x, out=None, flags: int = 0, reduce: bool = True, residual=None):
        """``residual`` (replicated, [*, N]): the block's ``x + linear(...)`` (examples/llama3_70b.py:160-162) folded into
        this linear.  The fused kernel adds it to the reduced sum; on the NCCL path rank 0 adds it to its partial, like
        the bias, so the sum counts it once."""
        sh = self.shard
        if reduce and self.size > 1 and self.fused is not None:
            return self.fused.matmul(x, sh.qweight, sh.qzeros, sh.scales, sh.g_idx, bits=sh.bits, bias=sh.bias, out=out, flags=flags,
                                     residual=residual)
        if residual is not None and self.rank == 0:
            from ..feedforward import quantized_matrix_multiply_residual
            partial = quantized_matrix_multiply_residual(x, sh.qweight, sh.qzeros, sh.scales, sh.g_idx, residual, bits=sh.bits,
                                                         bias=sh.bias, out=out, flags=flags)
        else:
            partial = self.shard.local_matmul(x, out=out, flags=flags)
        if reduce and self.size > 1:
            return self.all_reduce(partial)
        return partial

    def all_reduce(self, partial):
        from ..nccl.tensor import NCCLTensor
        version = self.communicator.version
        if isinstance(version, NCCLTensor):
            from ..nccl.dispatch import all_reduce_
            return all_reduce_(version, partial)
        return self.communicator.all_reduce(partial)
