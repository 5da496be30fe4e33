"""``dispatch(op, *tensors) -> tuple`` with the reference's call signature
(minit/core/dispatch.py:37-58), reduced to what the quantized-linear path needs: rules are
keyed by the operator class and tried highest priority first; a rule is a predicate on the
argument tuple.  There is no linear scan over unrelated operators and nothing is generated
at run time.

Two ways to register a rule:

* ``@register_dispatch(MatrixMultiply, predicate=..., priority=...)`` -- this package's own form: the operator
  class is named, the predicate sees the argument VALUES;
* ``@register_dispatch(predicate=..., priority=...)`` over a function with annotations -- the reference's form
  (minit/core/dispatch.py:52-58): the first parameter's annotation is the operator class (or a ``Union`` of
  them), the others are the accepted argument classes (``Union`` for several, ``*args: T`` for a variable tail);
  as in the reference the predicate of such a rule sees the argument TYPES.  Patterns are matched with
  ``isinstance``; parametrised patterns (``CollectiveTensor[CollectiveSpecSplit[Literal[0]]]``) are refused at
  registration, because matching them needs the reference's generic-type algebra -- use a predicate instead.
"""
from __future__ import annotations

import inspect
import typing
from typing import Callable, Dict, List, Optional, Tuple, Union

from .operator import Operator

_Rule = Tuple[int, Optional[Callable[..., bool]], Callable[..., tuple]]
_TABLE: Dict[type, List[_Rule]] = {}


_MERGED: Dict[type, List[_Rule]] = {}                        # per concrete operator class: its rules and its bases' rules, by priority


def _add_rule(op_type: type, priority: int, predicate, function) -> None:
    _TABLE.setdefault(op_type, []).append((priority, predicate, function))
    _MERGED.clear()


def _rules(op_type: type) -> List[_Rule]:
    rules = _MERGED.get(op_type)
    if rules is None:
        rules = [rule for base in op_type.__mro__ for rule in _TABLE.get(base, ())]   # a rule for a base class serves its subclasses
        rules.sort(key=lambda r: -r[0])                      # stable: the more specific class and the earlier rule win a tie
        _MERGED[op_type] = rules
    return rules


def _classes(annotation, what: str) -> Tuple[type, ...]:
    """the classes an annotation accepts: a class, or a Union / Optional of classes"""
    if annotation is inspect.Parameter.empty:
        raise TypeError(f"register_dispatch: {what} needs an annotation")
    if typing.get_origin(annotation) is Union:
        out: Tuple[type, ...] = ()
        for part in typing.get_args(annotation):
            out += _classes(part, what)
        return out
    if typing.get_origin(annotation) is not None or not isinstance(annotation, type):
        raise TypeError(f"register_dispatch: {what} is annotated {annotation!r}; only classes and Unions of classes "
                        "can be matched (give a predicate for anything finer)")
    return (annotation,)


def _from_annotations(function, predicate, priority: int) -> None:
    try:
        hints = typing.get_type_hints(function)              # resolves annotations written as strings
    except Exception:
        hints = {}                                           # names that cannot be resolved: take the annotations as they are
    parameters = list(inspect.signature(function).parameters.values())
    if not parameters:
        raise TypeError("register_dispatch: the rule takes the operator as its first parameter")
    fixed: List[Tuple[type, ...]] = []
    tail: Optional[Tuple[type, ...]] = None
    for parameter in parameters[1:]:
        annotation = hints.get(parameter.name, parameter.annotation)
        if parameter.kind is parameter.VAR_POSITIONAL:
            tail = _classes(annotation, f"*{parameter.name}")
        elif parameter.kind in (parameter.POSITIONAL_ONLY, parameter.POSITIONAL_OR_KEYWORD):
            fixed.append(_classes(annotation, parameter.name))
        else:
            raise TypeError(f"register_dispatch: parameter {parameter.name} must be positional")

    def accepts(*args) -> bool:
        if len(args) < len(fixed) or (len(args) > len(fixed) and tail is None):
            return False
        if not all(isinstance(arg, classes) for arg, classes in zip(args, fixed)):
            return False
        if not all(isinstance(arg, tail) for arg in args[len(fixed):]):
            return False
        return predicate is None or bool(predicate(*[type(arg) for arg in args]))

    first = parameters[0]
    for op_type in _classes(hints.get(first.name, first.annotation), first.name):
        if not issubclass(op_type, Operator):
            raise TypeError(f"register_dispatch: {op_type.__name__} is not an Operator")
        _add_rule(op_type, priority, accepts, function)


def register_dispatch(op_type: Optional[type] = None, *, predicate: Optional[Callable[..., bool]] = None, priority: int = 0):
    def decorator(function):
        if op_type is None:
            _from_annotations(function, predicate, priority)
        else:
            _add_rule(op_type, priority, predicate, function)
        return function
    return decorator


def dispatch(op: Operator, *args) -> tuple:
    for _, predicate, function in _rules(type(op)):
        if predicate is None or predicate(*args):
            outputs = function(op, *args)
            assert isinstance(outputs, tuple)
            return outputs
    raise TypeError(f"no implementation of {type(op).__name__} for {tuple(type(a).__name__ for a in args)}")
