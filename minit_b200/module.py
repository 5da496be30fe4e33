"""Minimal module container with the reference's buffer protocol (minit/module/module.py:11-72):
``register_buffer(name, shape, dtype)`` declares a slot and returns a placeholder,
``update_buffer(name, value)`` fills it (dotted names address children), calling the module
runs ``forward``."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
           "int32": torch.int32, "int8": torch.int8, "uint8": torch.uint8}


class BufferSpec:
    """Placeholder for a buffer that has not been loaded yet (shape + dtype only)."""

    def __init__(self, shape: Tuple[int, ...], dtype: str) -> None:
        self.shape = tuple(shape)
        self.dtype = dtype

    def __repr__(self) -> str:
        return f"BufferSpec({self.shape}, {self.dtype})"


class Module:
    def __init__(self) -> None:
        self.children: Dict[str, Any] = {}
        self.buffers: Dict[str, Tuple[Tuple[int, ...], str]] = {}

    def register_module(self, name: str, module):
        self.children[name] = ()
        return module

    def register_buffer(self, name: str, shape: Tuple[int, ...], dtype: str, buffer: Optional[torch.Tensor] = None):
        self.buffers[name] = (tuple(shape), dtype)
        return BufferSpec(shape, dtype) if buffer is None else buffer

    def named_buffers(self):
        for name in self.buffers:
            yield name, getattr(self, name)
        for module_name in self.children:
            for name, buffer in getattr(self, module_name).named_buffers():
                yield module_name + "." + name, buffer

    def get_child(self, name: str) -> "Module":
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            return self.get_child(prefix).get_child(suffix)
        assert name in self.children
        return getattr(self, name)

    def get_buffer(self, name: str):
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            return self.get_child(prefix).get_buffer(suffix)
        assert name in self.buffers
        return getattr(self, name)

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        """``sharded``: the value is a rank's part of the buffer (a ``CollectiveTensor`` or a torch shard produced by a
        loader epilogue): the dtype is still checked, the shape is the shard's own."""
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            self.get_child(prefix).update_buffer(suffix, value, sharded)
            return
        assert name in self.buffers, f"{name} is not a buffer of {type(self).__name__}"
        shape, dtype = self.buffers[name]
        if value.dtype != _DTYPES[dtype] or (not sharded and tuple(value.shape) != shape):
            raise ValueError(f"buffer {name}: expected {shape} {dtype}, got {tuple(value.shape)} {value.dtype}")
        setattr(self, name, value.contiguous() if isinstance(value, torch.Tensor) else value)

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)
