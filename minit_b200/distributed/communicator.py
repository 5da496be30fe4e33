"""DistributedCommunicator (reference: minit/distributed/communicator.py:15-50): every
collective threads a ``version`` token through dispatch, which both selects the backend
(the token's type) and orders the collectives."""
from __future__ import annotations

from ..core.dispatch import dispatch
from .operator import (DistributedAllGather, DistributedAllReduce, DistributedAllToAll, DistributedBroadcast,
                       DistributedRecv, DistributedReduceScatter, DistributedScatter, DistributedSend)


class DistributedCommunicator:
    def __init__(self, version) -> None:
        self.version = version

    def send(self, x, target: int):
        (self.version,) = dispatch(DistributedSend(target), self.version, x)

    def recv(self, source: int):
        (self.version, z) = dispatch(DistributedRecv(source), self.version)
        return z

    def broadcast(self, x, source: int):
        (self.version, z) = dispatch(DistributedBroadcast(source), self.version, x)
        return z

    def all_reduce(self, x):
        (self.version, z) = dispatch(DistributedAllReduce(), self.version, x)
        return z

    def all_gather(self, x, axis: int):
        (self.version, z) = dispatch(DistributedAllGather(axis), self.version, x)
        return z

    def reduce_scatter(self, x, axis: int):
        (self.version, z) = dispatch(DistributedReduceScatter(axis), self.version, x)
        return z

    def scatter(self, x, source: int, axis: int):
        (self.version, z) = dispatch(DistributedScatter(source, axis), self.version, x)
        return z

    def all_to_all(self, x, gather_axis: int, scatter_axis: int):
        (self.version, z) = dispatch(DistributedAllToAll(gather_axis, scatter_axis), self.version, x)
        return z
