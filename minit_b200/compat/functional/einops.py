"""``einsum`` and ``rearrange`` with the reference's equation syntax (minit/functional/einops.py:23-224): one letter per
axis, ``(ab)`` for an axis that is the product of a and b, ``...`` for the axes a term does not name, and a ``variables``
dictionary that supplies sizes the equation cannot infer and receives the sizes it does infer (callers reuse it to
undo a rearrangement).  The work is one reshape / permute / reshape (or one contraction) instead of the reference's
chain of expand, transpose and fold kernels."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch

from ..tensor import ScalarTensor
from .utils import integer, unwrap, wrap

__all__ = ["einsum", "rearrange"]

Term = Union[str, List[str]]


def _parse_term(term: str) -> List[Term]:
    dims: List[Term] = []
    i = 0
    while i < len(term):
        c = term[i]
        if c == "(":
            close = term.index(")", i)
            group = list(term[i + 1:close])
            assert all(s.isalpha() for s in group), f"bad group in {term!r}"
            dims.append(group)
            i = close + 1
        elif c == ".":
            assert term[i:i + 3] == "...", f"bad ellipsis in {term!r}"
            dims.append("...")
            i += 3
        else:
            assert c.isalpha(), f"bad axis name {c!r} in {term!r}"
            dims.append(c)
            i += 1
    return dims


def _parse(equation: str):
    inputs, output = equation.replace(" ", "").split("->")
    return [_parse_term(t) for t in inputs.split(",")], _parse_term(output)


def _expand_ellipsis(specs: Sequence[List[Term]], ranks: Sequence[Optional[int]]) -> None:
    names = None
    for spec, rank in zip(specs, ranks):
        if "..." in spec and rank is not None:
            assert names is None, "one term may carry the ellipsis"
            names = [f".{i}" for i in range(rank - (len(spec) - 1))]
    for spec in specs:
        if "..." in spec:
            assert names is not None
            i = spec.index("...")
            spec[i:i + 1] = names


def _flat(spec: Sequence[Term]) -> List[str]:
    out: List[str] = []
    for dim in spec:
        out.extend(dim) if isinstance(dim, list) else out.append(dim)
    return out


def _ungroup(spec: Sequence[Term], t: torch.Tensor, variables: Dict[str, object]) -> torch.Tensor:
    """t with every grouped axis split into its parts; records each axis size in ``variables``."""
    assert len(spec) == t.dim(), f"{len(spec)} axes named, tensor has {t.dim()}"
    sizes: List[int] = []
    for dim, size in zip(spec, t.shape):
        if isinstance(dim, list):
            known = 1
            unknown = None
            for sub in dim:
                if sub in variables:
                    known *= integer(variables[sub])
                else:
                    assert unknown is None, f"two unknown sizes in ({''.join(dim)})"
                    unknown = sub
            if unknown is not None:
                assert size % known == 0
                variables[unknown] = ScalarTensor(size // known, (), "int32")
            else:
                assert known == size, f"({''.join(dim)}) = {known}, axis has {size}"
            sizes.extend(integer(variables[sub]) for sub in dim)
        else:
            variables.setdefault(dim, ScalarTensor(size, (), "int32"))
            sizes.append(size)
    return t.reshape(sizes)


def _regroup(spec: Sequence[Term], t: torch.Tensor) -> torch.Tensor:
    shape: List[int] = []
    i = 0
    for dim in spec:
        n = len(dim) if isinstance(dim, list) else 1
        size = 1
        for s in t.shape[i:i + n]:
            size *= s
        shape.append(size)
        i += n
    return t.reshape(shape)


def _rearrange(input_spec, output_spec, t: torch.Tensor, variables: Dict[str, object]) -> torch.Tensor:
    t = _ungroup(input_spec, t, variables)
    names = _flat(input_spec)
    target = _flat(output_spec)
    assert all(name in target for name in names), "rearrange drops no axis"
    for name in target:                                   # axes the input does not have are broadcast
        if name not in names:
            names.append(name)
            t = t.unsqueeze(-1)
    t = t.permute([names.index(name) for name in target])
    t = t.expand([integer(variables[name]) if t.shape[i] == 1 and name in variables else t.shape[i] for i, name in enumerate(target)])
    return _regroup(output_spec, t)


def rearrange(equation: str, x, variables: Optional[Dict[str, object]] = None):
    if variables is None:
        variables = {}
    input_specs, output_spec = _parse(equation)
    assert len(input_specs) == 1
    _expand_ellipsis([input_specs[0], output_spec], [len(x._shape), None])
    for i in range(len(input_specs[0]), len(x._shape)):   # trailing axes the equation does not name stay where they are
        input_specs[0].append(f"+{i}")                    # (the embedding lookup of the examples relies on it)
        output_spec.append(f"+{i}")
    return wrap(_rearrange(input_specs[0], output_spec, unwrap(x), variables))


def einsum(equation: str, *args, variables: Optional[Dict[str, object]] = None):
    if variables is None:
        variables = {}
    input_specs, output_spec = _parse(equation)
    assert len(input_specs) == len(args)
    _expand_ellipsis([*input_specs, output_spec], [len(arg._shape) for arg in args] + [None])
    operands = [_ungroup(spec, unwrap(arg), variables) for spec, arg in zip(input_specs, args)]
    letters: Dict[str, str] = {}
    pool = iter("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ")

    def term(names: Sequence[str]) -> str:
        return "".join(letters.setdefault(name, next(pool)) for name in names)

    lhs = ",".join(term(_flat(spec)) for spec in input_specs)
    z = torch.einsum(f"{lhs}->{term(_flat(output_spec))}", *operands)
    return wrap(_regroup(output_spec, z))
