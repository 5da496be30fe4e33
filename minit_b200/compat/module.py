"""``Module`` / ``ModuleList`` for models written against the reference (minit/module/module.py:11-72,
minit/module/list.py:6-24): buffers are declared with a shape and a dtype name, start as ``MetaTensor`` placeholders
and are filled by ``update_buffer`` -- here with ``CUDATensor`` values, so a checkpoint loader that hands over torch
tensors (``minit_b200.checkpoint``) feeds the same models."""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch

from ..module import Module as _TorchModule
from .tensor import CUDATensor, MetaTensor, Tensor, to_immediate_shape


class Module(_TorchModule):
    def __class_getitem__(cls, item):                        # annotations such as ``ModuleList[Block]`` (the reference's classes are Generic)
        return cls

    def register_buffer(self, name: str, shape: Tuple[int, ...], dtype: str, buffer: Optional[Tensor] = None):
        self.buffers[name] = (to_immediate_shape(shape), dtype)
        return MetaTensor(shape, dtype) if buffer is None else buffer

    def get_buffer(self, name: str):
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            return self.get_child(prefix).get_buffer(suffix)
        assert name in self.buffers, f"{name} is not a buffer of {type(self).__name__}"
        return self[int(name)] if name[0].isdigit() else getattr(self, name)

    def get_child(self, name: str):
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            return self.get_child(prefix).get_child(suffix)
        assert name in self.children, f"{name} is not a child of {type(self).__name__}"
        return self[int(name)] if name[0].isdigit() else getattr(self, name)

    def named_buffers(self):
        for name in self.buffers:
            yield name, self.get_buffer(name)
        for module_name in self.children:
            for name, buffer in self.get_child(module_name).named_buffers():
                yield module_name + "." + name, buffer

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        if "." in name:
            prefix, suffix = name.split(".", maxsplit=1)
            self.get_child(prefix).update_buffer(suffix, value, sharded)
            return
        assert name in self.buffers, f"{name} is not a buffer of {type(self).__name__}"
        shape, dtype = self.buffers[name]
        if isinstance(value, torch.Tensor):
            value = CUDATensor.from_torch(value)
        if isinstance(value, Tensor):
            if value.dtype != dtype or (not sharded and to_immediate_shape(value.shape) != tuple(shape)):
                raise ValueError(f"buffer {name}: expected {tuple(shape)} {dtype}, got {to_immediate_shape(value.shape)} {value.dtype}")
        if name[0].isdigit():
            self[int(name)] = value
        else:
            setattr(self, name, value)


class ModuleList(Module):
    def __init__(self) -> None:
        super().__init__()
        self._module_list: List[Module] = []

    def append(self, module) -> None:
        self._module_list.append(self.register_module(str(len(self._module_list)), module))

    def __getitem__(self, index):
        return self._module_list[index]

    def __iter__(self) -> Iterator:
        return iter(self._module_list)

    def __len__(self) -> int:
        return len(self._module_list)
