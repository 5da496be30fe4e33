"""Placement specs of a tensor across the world group (reference: minit/collective/spec.py:12-44)."""
from dataclasses import dataclass


@dataclass(frozen=True)
class CollectiveSpecSplit:
    axis: int


@dataclass(frozen=True)
class CollectiveSpecPartial:
    pass


@dataclass(frozen=True)
class CollectiveSpecBroadcast:
    pass


@dataclass(frozen=True)
class CollectiveSpecUnique:
    rank: int
