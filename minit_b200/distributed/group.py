"""World group bookkeeping (reference: minit/distributed/group.py:5-21)."""
from dataclasses import dataclass


@dataclass(frozen=True)
class DistributedGroup:
    size: int
    rank: int


_WORLD = None


def get_world() -> DistributedGroup:
    return _WORLD


def initialize_world(rank: int, size: int):
    global _WORLD
    assert _WORLD is None, "the world group is initialised once per process"
    assert 0 <= rank < size
    _WORLD = DistributedGroup(size, rank)


def reset_world():
    """Forget the world group (tests that start several worlds in one process)."""
    global _WORLD
    _WORLD = None
