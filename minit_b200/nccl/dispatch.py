"""NCCL implementations of the three collectives the reference implements
(minit/nccl/dispatch.py:11-50).  Differences: they run on the caller's current CUDA stream
instead of the null stream, and all_reduce works in place when asked to (``x`` is both
buffers), which is how the row-parallel linear uses it."""
from __future__ import annotations

import torch

from .. import _lib
from ..core.dispatch import register_dispatch
from ..distributed.group import get_world
from ..distributed.operator import DistributedAllGather, DistributedAllReduce, DistributedBroadcast
from .tensor import NCCLTensor

_NCCL_DTYPE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2, torch.int32: 3}


def _is_nccl(version, *args):
    return isinstance(version, NCCLTensor)


@register_dispatch(DistributedAllGather, predicate=_is_nccl)
def dispatch_all_gather(op: DistributedAllGather, version: NCCLTensor, x: torch.Tensor):
    if op.axis != 0:
        x = x.transpose(0, op.axis).contiguous()
    dev = _lib.require_cuda(x)
    z = torch.empty((x.shape[0] * get_world().size, *x.shape[1:]), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.nccl_all_gather(_lib.current_stream(dev), version.comm, x.data_ptr(), z.data_ptr(), x.numel(),
                                      _NCCL_DTYPE[x.dtype])
    _lib.check(rc, "nccl_all_gather")
    if op.axis != 0:
        z = z.transpose(0, op.axis).contiguous()
    return (version, z)


@register_dispatch(DistributedAllReduce, predicate=_is_nccl)
def dispatch_all_reduce(op: DistributedAllReduce, version: NCCLTensor, x: torch.Tensor, out: torch.Tensor = None):
    dev = _lib.require_cuda(x)
    z = torch.empty_like(x) if out is None else out
    with torch.cuda.device(dev):
        rc = _lib.lib.nccl_all_reduce(_lib.current_stream(dev), version.comm, x.data_ptr(), z.data_ptr(), x.numel(),
                                      _NCCL_DTYPE[x.dtype])
    _lib.check(rc, "nccl_all_reduce")
    return (version, z)


@register_dispatch(DistributedBroadcast, predicate=_is_nccl)
def dispatch_broadcast(op: DistributedBroadcast, version: NCCLTensor, x: torch.Tensor):
    dev = _lib.require_cuda(x)
    z = torch.empty_like(x)
    with torch.cuda.device(dev):
        rc = _lib.lib.nccl_broadcast(_lib.current_stream(dev), version.comm, x.data_ptr(), z.data_ptr(), x.numel(),
                                     _NCCL_DTYPE[x.dtype], op.source)
    _lib.check(rc, "nccl_broadcast")
    return (version, z)


def all_reduce_(version: NCCLTensor, x: torch.Tensor) -> torch.Tensor:
    """In-place sum over ranks on the current stream (no allocation; safe inside CUDA graph capture)."""
    dispatch_all_reduce(DistributedAllReduce(), version, x, out=x)
    return x
