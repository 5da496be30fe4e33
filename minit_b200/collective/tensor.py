"""CollectiveTensor: a local shard plus how it relates to the global tensor
(reference: minit/collective/tensor.py:16-111).  Conversions follow the reference:
Split -> all_gather, Partial -> all_reduce, Unique -> broadcast; to_split is a local slice."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..distributed.communicator import DistributedCommunicator
from ..distributed.group import get_world
from .spec import CollectiveSpecBroadcast, CollectiveSpecPartial, CollectiveSpecSplit, CollectiveSpecUnique


class CollectiveTensor:
    __slots__ = ["_communicator", "_shape", "_local", "_spec"]

    def __init__(self, communicator: DistributedCommunicator, local: Optional[torch.Tensor], spec, shape: Tuple[int, ...]) -> None:
        assert not isinstance(local, CollectiveTensor)
        self._communicator = communicator
        self._local = local
        self._spec = spec
        self._shape = tuple(shape)

    @property
    def shape(self):
        return self._shape

    @property
    def dtype(self):
        return self._local.dtype

    @property
    def spec(self):
        return self._spec

    @property
    def device(self):
        return self._local.device

    def dim(self):
        return len(self._shape)

    @staticmethod
    def from_broadcast(communicator, local) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecBroadcast(), local.shape)

    @staticmethod
    def from_split(communicator, local, axis: int) -> "CollectiveTensor":
        shape = tuple(local.shape)
        shape = shape[:axis] + (shape[axis] * get_world().size,) + shape[axis + 1:]
        return CollectiveTensor(communicator, local, CollectiveSpecSplit(axis), shape)

    @staticmethod
    def from_unique(communicator, local, rank: int) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecUnique(rank), local.shape)

    @staticmethod
    def from_partial(communicator, local) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecPartial(), local.shape)

    def to_broadcast(self) -> "CollectiveTensor":
        spec = self._spec
        if isinstance(spec, CollectiveSpecBroadcast):
            return self
        if isinstance(spec, CollectiveSpecSplit):
            return CollectiveTensor.from_broadcast(self._communicator, self._communicator.all_gather(self._local, spec.axis))
        if isinstance(spec, CollectiveSpecPartial):
            return CollectiveTensor.from_broadcast(self._communicator, self._communicator.all_reduce(self._local))
        if isinstance(spec, CollectiveSpecUnique):
            return CollectiveTensor.from_broadcast(self._communicator, self._communicator.broadcast(self._local, spec.rank))
        raise AssertionError(spec)

    def to_partial(self) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecPartial):
            return self
        full = self.to_broadcast()
        return CollectiveTensor.from_partial(self._communicator, full._local / get_world().size)

    def to_split(self, axis: int) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecSplit) and self._spec.axis == axis:
            return self
        full = self.to_broadcast()
        world = get_world()
        assert full._shape[axis] % world.size == 0
        size = full._shape[axis] // world.size
        local = full._local.narrow(axis, size * world.rank, size).contiguous()
        return CollectiveTensor.from_split(self._communicator, local, axis)

    def to_unique(self, rank: int) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecUnique) and self._spec.rank == rank:
            return self
        full = self.to_broadcast()
        return CollectiveTensor.from_unique(self._communicator, full._local, rank)

    def numpy(self):
        return self.to_broadcast()._local.cpu().numpy()
