"""``CollectiveTensor`` for models written against the reference's Python surface: a rank's local tensor plus its
placement across the world group (minit/collective/tensor.py:16-111), with the tensor method surface of
``compat.tensor.Tensor``, so that a model whose inputs and weights are wrapped this way runs tensor-parallel unchanged.

Two rules carry the reference's behaviour (minit/collective/dispatch.py:13-44):

* any functional operator that meets a ``CollectiveTensor`` works on whole tensors: every collective argument is
  brought to the broadcast placement (all-gather of a split, all-reduce of a partial, broadcast of a unique one), the
  operator runs locally and its results are broadcast-placed (``collective_aware`` wraps the functional layer);
* ``matrix_multiply(x, w)`` with a weight split along its rows (output features) keeps the product split along the
  last axis, and with a weight split along its columns (input features) multiplies the matching slice of x and leaves
  a partial sum -- the column- and row-parallel linears.  A ``ShardedQuantized`` weight (a rank's shard of a GPTQ
  tensor, ``minit_b200.collective``) follows the same two rules with the fused kernels as the local product.

The local tensor may be a torch tensor (what a checkpoint loader's epilogue receives) or one of this layer's tensors;
collectives always run on torch tensors through ``DistributedCommunicator``."""
from __future__ import annotations

import functools
from typing import Optional

import torch

from ..collective.spec import CollectiveSpecBroadcast, CollectiveSpecPartial, CollectiveSpecSplit, CollectiveSpecUnique
from ..collective.tensor import CollectiveTensor as _TorchCollectiveTensor
from ..distributed.group import get_world
from .tensor import CUDATensor, ScalarTensor, Tensor, dtype_name, to_immediate_shape, to_symbolic_shape


def _compat(local):
    return CUDATensor.from_torch(local) if isinstance(local, torch.Tensor) else local


def _torch(local) -> torch.Tensor:
    if isinstance(local, CUDATensor):
        return local.as_torch()
    assert isinstance(local, torch.Tensor), f"a collective needs a device tensor, got {type(local).__name__}"
    return local


class CollectiveTensor(_TorchCollectiveTensor, Tensor):
    __slots__ = ()

    def __init__(self, communicator, local, spec, shape) -> None:
        assert not isinstance(local, _TorchCollectiveTensor)
        self._communicator, self._local, self._spec = communicator, local, spec
        self._shape = to_immediate_shape(shape)

    @property
    def shape(self):
        return tuple(CollectiveTensor.from_broadcast(self._communicator, dim) for dim in to_symbolic_shape(self._shape))

    @property
    def dtype(self) -> str:
        dtype = self._local.dtype
        return dtype if isinstance(dtype, str) else dtype_name(dtype)

    @property
    def device(self):
        return self._local.device

    def type(self):
        return CollectiveTensor

    # ---- placements -----------------------------------------------------------------------------------------------
    @staticmethod
    def from_broadcast(communicator, local) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecBroadcast(), local.shape)

    @staticmethod
    def from_split(communicator, local, axis: int) -> "CollectiveTensor":
        shape = list(to_immediate_shape(local.shape))
        shape[axis] *= get_world().size
        return CollectiveTensor(communicator, local, CollectiveSpecSplit(axis), shape)

    @staticmethod
    def from_unique(communicator, local, rank: int) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecUnique(rank), local.shape)

    @staticmethod
    def from_partial(communicator, local) -> "CollectiveTensor":
        return CollectiveTensor(communicator, local, CollectiveSpecPartial(), local.shape)

    def local(self):
        """this rank's tensor in the broadcast placement, as one of this layer's tensors"""
        return _compat(self.to_broadcast()._local)

    def to_broadcast(self) -> "CollectiveTensor":
        spec, comm = self._spec, self._communicator
        if isinstance(spec, CollectiveSpecBroadcast):
            return self
        if isinstance(spec, CollectiveSpecSplit):
            whole = comm.all_gather(_torch(self._local), spec.axis)
        elif isinstance(spec, CollectiveSpecPartial):
            whole = comm.all_reduce(_torch(self._local))
        elif isinstance(spec, CollectiveSpecUnique):
            whole = comm.broadcast(_torch(self._local), spec.rank)
        else:
            raise AssertionError(spec)
        return CollectiveTensor.from_broadcast(comm, _compat(whole))

    def to_split(self, axis: int) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecSplit) and self._spec.axis == axis:
            return self
        whole = _torch(self.to_broadcast()._local)
        world = get_world()
        assert whole.shape[axis] % world.size == 0, f"axis {axis} of {tuple(whole.shape)} does not divide by {world.size}"
        size = whole.shape[axis] // world.size
        return CollectiveTensor.from_split(self._communicator, _compat(whole.narrow(axis, size * world.rank, size).contiguous()), axis)

    def to_partial(self) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecPartial):
            return self
        whole = _torch(self.to_broadcast()._local)
        return CollectiveTensor.from_partial(self._communicator, _compat(whole / get_world().size))

    def to_unique(self, rank: int) -> "CollectiveTensor":
        if isinstance(self._spec, CollectiveSpecUnique) and self._spec.rank == rank:
            return self
        return CollectiveTensor.from_unique(self._communicator, self.to_broadcast()._local, rank)

    def numpy(self):
        return self.local().numpy()

    def item(self):
        assert isinstance(self._spec, CollectiveSpecBroadcast)
        return self._local.item()

    def __index__(self) -> int:
        return int(self.item())

    def __bool__(self) -> bool:
        return bool(self.item())

    def __repr__(self) -> str:
        return f"CollectiveTensor({self._shape}, {self.dtype}, {self._spec})"


# ---- the functional layer on collective tensors -----------------------------------------------------------------------
def _communicator_of(value) -> Optional[object]:
    if isinstance(value, CollectiveTensor):
        return value._communicator
    if isinstance(value, (list, tuple)):
        for item in value:
            found = _communicator_of(item)
            if found is not None:
                return found
    if isinstance(value, dict):
        return _communicator_of(list(value.values()))
    return None


def _localise(value):
    if isinstance(value, CollectiveTensor):
        return value.local()
    if isinstance(value, (list, tuple)):
        return type(value)(_localise(item) for item in value)
    return value


def _place(communicator, value):
    if isinstance(value, Tensor) and not isinstance(value, CollectiveTensor):
        return CollectiveTensor.from_broadcast(communicator, value)
    if isinstance(value, tuple):
        return tuple(_place(communicator, item) for item in value)
    return value


def collective_aware(function):
    """The generic rule: collective arguments are gathered, the operator runs on whole tensors, results are broadcast-placed."""
    @functools.wraps(function)
    def wrapper(*args, **kwargs):
        communicator = _communicator_of(args) or _communicator_of(kwargs)
        if communicator is None:
            return function(*args, **kwargs)
        if "variables" in kwargs and isinstance(kwargs["variables"], dict):      # einops: sizes in, inferred sizes out
            kwargs["variables"].update({k: _localise(v) for k, v in kwargs["variables"].items()})
        local_args = [_localise(arg) if not isinstance(arg, dict) else arg for arg in args]
        for arg in local_args:
            if isinstance(arg, dict):
                arg.update({k: _localise(v) for k, v in arg.items()})
        local_kwargs = {k: (v if isinstance(v, dict) else _localise(v)) for k, v in kwargs.items()}
        return _place(communicator, function(*local_args, **local_kwargs))
    return wrapper


def matrix_multiply(x, y, local_product):
    """The placement rules of a linear layer; ``local_product(x, w)`` multiplies this layer's tensors."""
    communicator = _communicator_of((x, y))
    if communicator is None:
        raise TypeError("a sharded weight needs a CollectiveTensor input (its communicator places the result)")
    if not isinstance(x, CollectiveTensor):
        x = CollectiveTensor.from_broadcast(communicator, x)
    lead = x._shape[:-1]
    from ..collective.quantized import ShardedQuantized
    if isinstance(y, ShardedQuantized):                                        # a rank's shard of a GPTQ weight: the fused kernels
        def fused(xt: torch.Tensor) -> CUDATensor:
            z = y.local_matmul(xt.reshape(-1, xt.shape[-1]))
            return CUDATensor.from_torch(z.reshape(*xt.shape[:-1], z.shape[-1]))
        if y.mode == "column":
            return CollectiveTensor.from_split(communicator, fused(_torch(x.local())), len(lead))
        return CollectiveTensor.from_partial(communicator, fused(_torch(x.to_split(len(lead))._local)))
    spec = y._spec if isinstance(y, CollectiveTensor) else None
    if isinstance(spec, CollectiveSpecSplit) and spec.axis == 0:               # column-parallel: the outputs stay split
        z = local_product(x.local(), _compat(y._local))
        return CollectiveTensor.from_split(communicator, z, len(lead))
    if isinstance(spec, CollectiveSpecSplit) and spec.axis == 1:               # row-parallel: a partial sum
        xs = x.to_split(len(lead))
        return CollectiveTensor.from_partial(communicator, local_product(_compat(xs._local), _compat(y._local)))
    w = y.local() if isinstance(y, CollectiveTensor) else y
    return CollectiveTensor.from_broadcast(communicator, local_product(x.local(), w))
