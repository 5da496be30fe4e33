"""``dispatch(op, *tensors) -> tuple`` with the reference's call signature
(minit/core/dispatch.py:37-58), reduced to what the quantized-linear path needs: rules are
keyed by the operator class and tried highest priority first; a rule is a predicate on the
argument tuple.  There is no signature introspection, no linear scan over unrelated
operators and nothing is generated at run time.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

from .operator import Operator

_Rule = Tuple[int, Optional[Callable[..., bool]], Callable[..., tuple]]
_TABLE: Dict[type, List[_Rule]] = {}


def register_dispatch(op_type: type, *, predicate: Optional[Callable[..., bool]] = None, priority: int = 0):
    def decorator(function):
        rules = _TABLE.setdefault(op_type, [])
        rules.append((priority, predicate, function))
        rules.sort(key=lambda r: -r[0])
        return function
    return decorator


def dispatch(op: Operator, *args) -> tuple:
    for _, predicate, function in _TABLE.get(type(op), ()):
        if predicate is None or predicate(*args):
            outputs = function(op, *args)
            assert isinstance(outputs, tuple)
            return outputs
    raise TypeError(f"no implementation of {type(op).__name__} for {tuple(type(a).__name__ for a in args)}")
