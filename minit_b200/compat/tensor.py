"""The reference's tensor types on torch storage, for code written against MiniT's Python surface.

``Tensor`` carries the method surface of minit/core/array.py:13-239 (every method forwards to the function
of the same name in ``functional``), ``ScalarTensor`` is the host-side scalar of minit/core/scalar.py:8-43,
``MetaTensor`` the shape-and-dtype placeholder of minit/core/meta.py:7-28 and ``CUDATensor`` the device
tensor of minit/cuda/tensor.py:15-131: a shape, a dtype name and a block of device memory that views
(``add_axis``, ``fold``, ``expand``, ``reinterpret``) share.  The memory is a torch byte tensor; nothing here
is on the quantized-linear hot path, which is reached through ``functional.matrix_multiply`` with a
``QuantizedTensor`` operand.
"""
from __future__ import annotations

from numbers import Number
from typing import Optional, Sequence, Tuple

import numpy
import torch

# name -> (torch dtype, python type, bytes): minit/core/dtype.py:39-49 plus the boolean the comparisons return
_DTYPES = {
    "float64": (torch.float64, float, 8), "float32": (torch.float32, float, 4),
    "float16": (torch.float16, float, 2), "bfloat16": (torch.bfloat16, float, 2),
    "int64": (torch.int64, int, 8), "int32": (torch.int32, int, 4), "int16": (torch.int16, int, 2), "int8": (torch.int8, int, 1),
    "uint64": (torch.uint64, int, 8), "uint32": (torch.uint32, int, 4), "uint16": (torch.uint16, int, 2), "uint8": (torch.uint8, int, 1),
    "bool": (torch.bool, bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

_device: Optional[torch.device] = None


def set_device(device) -> None:
    """Where ``CUDATensor`` memory lives.  The default is the current CUDA device; a host device can be set to
    exercise the glue (shapes, einops, modules) without a GPU -- the quantized product still needs one."""
    global _device
    _device = None if device is None else torch.device(device)


def current_device() -> torch.device:
    if _device is not None:
        return _device
    if not torch.cuda.is_available():
        raise RuntimeError("minit_b200.compat: no CUDA device (set_device('cpu') runs the glue on the host)")
    return torch.device("cuda", torch.cuda.current_device())


def torch_dtype(name: str) -> torch.dtype:
    return _DTYPES[name][0]


def dtype_name(dtype: torch.dtype) -> str:
    return _NAMES[dtype]


def dtype_size(name: str) -> int:
    return _DTYPES[name][2]


def python_type(name: str) -> type:
    return _DTYPES[name][1]


class DataTypeInfo:
    """minit/core/dtype.py:5-20"""
    __slots__ = ("name", "python_type", "size_in_bytes")

    def __init__(self, name: str) -> None:
        self.name, self.python_type, self.size_in_bytes = name, _DTYPES[name][1], _DTYPES[name][2]


def dtype_info(name: str) -> DataTypeInfo:
    return DataTypeInfo(name)


class Tensor:
    """Method surface of the reference's arrays; operators map to the functional layer."""

    @property
    def shape(self) -> Tuple["Tensor", ...]:
        raise NotImplementedError()

    @property
    def dtype(self) -> str:
        raise NotImplementedError()

    @property
    def device(self) -> str:
        raise NotImplementedError()

    def type(self):
        return type(self)

    @property
    def size(self):
        total = ScalarTensor(1, (), "int32")
        for dim in self.shape:
            total = total * dim
        return total

    def __getitem__(self, index):
        assert not isinstance(index, tuple)
        if isinstance(index, slice):
            assert index.step is None
            if index.start is None and index.stop is None:
                return self
            start = 0 if index.start is None else index.start
            stop = self.shape[0] if index.stop is None else index.stop
            return self.slice(start, stop, 0)
        return self.slice(index, index + 1, 0).remove_axis(0)

    __hash__ = object.__hash__


def _forward(name: str, module: str):
    def method(self, *args, **kwargs):
        from . import functional
        return getattr(getattr(functional, module), name)(self, *args, **kwargs)
    method.__name__ = name
    return method


def _reflected(name: str, module: str):
    def method(self, other):
        from . import functional
        return getattr(getattr(functional, module), name)(other, self)
    return method


for _module, _names in {
    "shape": ("fold", "expand", "add_axis", "remove_axis", "broadcast", "transpose", "repeat", "repeat_interleaved", "reinterpret"),
    "reduce": ("sum", "mean", "max"),
    "index": ("slice", "slice_set", "index", "index_set", "split"),
    "arith": ("add", "subtract", "multiply", "divide", "floor_divide", "modulo", "power", "exponential", "logarithm", "square",
              "square_root", "sine", "cosine", "cast", "greater_than", "less_than", "greater_equal", "less_equal", "equal",
              "not_equal", "logical_not", "logical_and", "logical_or"),
}.items():
    for _name in _names:
        setattr(Tensor, _name, _forward(_name, _module))
for _dunder, _name in {"add": "add", "sub": "subtract", "mul": "multiply", "truediv": "divide", "floordiv": "floor_divide",
                       "mod": "modulo", "pow": "power"}.items():
    setattr(Tensor, f"__{_dunder}__", _forward(_name, "arith"))
    setattr(Tensor, f"__r{_dunder}__", _reflected(_name, "arith"))
for _dunder, _name in {"gt": "greater_than", "lt": "less_than", "ge": "greater_equal", "le": "less_equal", "eq": "equal",
                       "ne": "not_equal", "and": "logical_and", "or": "logical_or"}.items():
    setattr(Tensor, f"__{_dunder}__", _forward(_name, "arith"))


def _rearrange(self, equation: str, variables=None):
    from .functional.einops import rearrange
    return rearrange(equation, self, variables)


Tensor.rearrange = _rearrange


class ScalarTensor(Tensor):
    """One number on the host with a dtype name: tensor dimensions, offsets, constants."""
    __slots__ = ("_value", "_shape", "_dtype")

    def __init__(self, value: Number, shape: Tuple = (), dtype: str = "int32") -> None:
        assert not isinstance(value, Tensor) and dtype in _DTYPES
        self._value, self._shape, self._dtype = value, tuple(shape), dtype

    @property
    def shape(self):
        return self._shape

    @property
    def dtype(self) -> str:
        return self._dtype

    @property
    def device(self) -> str:
        return "host"

    def value(self):
        return self._value

    def item(self):
        assert len(self._shape) == 0
        return python_type(self._dtype)(self._value)

    def numpy(self):
        return numpy.full((), self._value, dtype=self._dtype if self._dtype != "bfloat16" else "float32")

    def __index__(self) -> int:
        assert python_type(self._dtype) is int
        return int(self._value)

    def __int__(self) -> int:
        return int(self._value)

    def __float__(self) -> float:
        return float(self._value)

    def __bool__(self) -> bool:
        return bool(self._value)

    def __repr__(self) -> str:
        return f"Scalar({self._value}: {self._dtype})"


def to_immediate_shape(shape: Sequence) -> Tuple[int, ...]:
    """minit/core/shape.py:12-13"""
    return tuple(dim.item() if isinstance(dim, Tensor) else int(dim) for dim in shape)


def to_symbolic_shape(shape: Sequence) -> Tuple[Tensor, ...]:
    """minit/core/shape.py:16-17"""
    return tuple(dim if isinstance(dim, Tensor) else ScalarTensor(dim, (), "int32") for dim in shape)


class MetaTensor(Tensor):
    """Shape and dtype only: what ``Module.register_buffer`` hands out until a checkpoint fills the buffer."""

    def __init__(self, shape: Sequence, dtype: str) -> None:
        self._shape, self._dtype = tuple(shape), dtype

    @property
    def shape(self):
        return to_symbolic_shape(self._shape)

    @property
    def dtype(self) -> str:
        return self._dtype

    @property
    def device(self) -> str:
        return "meta"

    def __repr__(self) -> str:
        return f"MetaTensor({to_immediate_shape(self._shape)}, {self._dtype})"


class CUDAMemory:
    """A block of device bytes (``_pointer``, ``_size``, ``reset()`` as in the reference's allocator)."""
    __slots__ = ("_bytes",)

    def __init__(self, size: int, storage: Optional[torch.Tensor] = None) -> None:
        self._bytes = torch.empty(int(size), dtype=torch.uint8, device=current_device()) if storage is None else storage

    @property
    def _pointer(self) -> int:
        return self._bytes.data_ptr()

    @property
    def _size(self) -> int:
        return self._bytes.numel()

    def reset(self) -> None:
        self._bytes.zero_()


def _count(shape: Sequence[int]) -> int:
    total = 1
    for dim in shape:
        assert isinstance(dim, int), f"immediate shape expected, got {dim!r}"
        total *= dim
    return total


class CUDATensor(Tensor):
    __slots__ = ("_memory", "_shape", "_item", "_dtype")

    def __init__(self, shape: Tuple[int, ...], dtype: str) -> None:
        self._memory: Optional[CUDAMemory] = None
        self._item: Optional[Number] = None
        self._shape = tuple(shape)
        self._dtype = dtype

    # ---- the reference's surface -------------------------------------------------------------------------------
    @property
    def shape(self) -> Tuple[Tensor, ...]:
        return tuple(ScalarTensor(dim, (), "int32") for dim in self._shape)

    @property
    def dtype(self) -> str:
        return self._dtype

    @property
    def device(self) -> str:
        return "cuda"

    @property
    def memory(self) -> CUDAMemory:
        if self._memory is None and self._item is not None:
            self._memory = CUDAMemory(dtype_size(self._dtype))
            self.as_torch().fill_(self._item)
        return self._memory

    @property
    def data_ptr(self) -> int:
        return self.memory._pointer

    @staticmethod
    def allocate(shape: Tuple[int, ...], dtype: str) -> "CUDATensor":
        result = CUDATensor(tuple(shape), dtype)
        result._memory = CUDAMemory(dtype_size(dtype) * _count(shape))
        return result

    @staticmethod
    def wrap(shape: Tuple[int, ...], dtype: str, memory: CUDAMemory) -> "CUDATensor":
        assert memory._size == dtype_size(dtype) * _count(shape)
        result = CUDATensor(tuple(shape), dtype)
        result._memory = memory
        return result

    @staticmethod
    def from_numpy(array) -> "CUDATensor":
        dtype = str(array.dtype).split(".")[-1]
        result = CUDATensor.allocate(tuple(array.shape), dtype)
        result.copy_from_numpy(array)
        return result

    @staticmethod
    def from_item(item: Number, dtype: str) -> "CUDATensor":
        result = CUDATensor((), dtype)
        result._item = item
        return result

    def copy_from_numpy(self, array) -> None:
        assert tuple(array.shape) == self._shape, f"{tuple(array.shape)} vs {self._shape}"
        source = array if isinstance(array, torch.Tensor) else torch.from_numpy(numpy.ascontiguousarray(array))
        assert dtype_name(source.dtype) == self._dtype
        self.as_torch().copy_(source)

    def numpy(self):
        host = self.as_torch().cpu()
        if host.dtype == torch.bfloat16:                      # numpy has no bfloat16
            host = host.float()
        return host.numpy()

    def item(self):
        if self._item is not None:
            return python_type(self._dtype)(self._item)
        return self.as_torch().item()

    # ---- torch side ----------------------------------------------------------------------------------------------
    def as_torch(self) -> torch.Tensor:
        """The typed view of this tensor's memory (shares it)."""
        return self.memory._bytes.view(torch_dtype(self._dtype)).view(self._shape)

    @staticmethod
    def from_torch(tensor: torch.Tensor) -> "CUDATensor":
        """Adopts a torch tensor without a copy when it is contiguous and already on the device."""
        device = current_device()
        tensor = tensor.detach().to(device).contiguous()
        result = CUDATensor(tuple(tensor.shape), dtype_name(tensor.dtype))
        result._memory = CUDAMemory(0, tensor.reshape(-1).view(torch.uint8))
        return result

    def __repr__(self) -> str:
        return f"CUDATensor({self._shape}, {self._dtype})"


def as_torch(x):
    """torch view of a device tensor; torch tensors pass through."""
    return x.as_torch() if isinstance(x, CUDATensor) else x
