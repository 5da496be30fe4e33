"""Version token backed by a torch.distributed process group: the same three collectives as
the NCCL backend, on whatever backend the group was created with (``nccl`` on GPUs, ``gloo``
for the CPU ranks that test the sharding logic without a GPU)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..core.dispatch import register_dispatch
from .operator import DistributedAllGather, DistributedAllReduce, DistributedBroadcast


class TorchDistTensor:
    def __init__(self, group=None) -> None:
        self.group = group

    @property
    def shape(self):
        return ()

    @property
    def dtype(self):
        return "int64"

    @property
    def device(self):
        return "torch.distributed"


def _is_td(version, *args):
    return isinstance(version, TorchDistTensor)


@register_dispatch(DistributedAllGather, predicate=_is_td)
def _all_gather(op: DistributedAllGather, version: TorchDistTensor, x: torch.Tensor):
    size = dist.get_world_size(version.group)
    parts = [torch.empty_like(x) for _ in range(size)]
    dist.all_gather(parts, x.contiguous(), group=version.group)
    return (version, torch.cat(parts, dim=op.axis))


@register_dispatch(DistributedAllReduce, predicate=_is_td)
def _all_reduce(op: DistributedAllReduce, version: TorchDistTensor, x: torch.Tensor):
    z = x.clone()
    dist.all_reduce(z, op=dist.ReduceOp.SUM, group=version.group)
    return (version, z)


@register_dispatch(DistributedBroadcast, predicate=_is_td)
def _broadcast(op: DistributedBroadcast, version: TorchDistTensor, x: torch.Tensor):
    z = x.clone()
    dist.broadcast(z, src=op.source, group=version.group)
    return (version, z)
