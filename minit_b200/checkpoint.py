"""Checkpoint ingest with the reference's entry points (minit/module/checkpoint.py:11-47):
``load_from_torch``, ``load_from_safetensors``, ``load_from_safetensors_index``.  Each tensor of a file
goes to the module buffer of the same dotted name, cast to the buffer's dtype and checked against its
shape, after an optional ``epilogue(name, tensor)`` (the hook the reference's tensor-parallel servers
use to shard while loading, examples/llama3_70b.py:298-310).

Differences: tensors land on ``device`` (the kernels take CUDA tensors only); the safetensors container
is parsed here (8-byte little-endian header length, JSON header, raw little-endian data), so the
``safetensors`` package is not needed; GPTQ layers with act-order are sorted by group on their first
call (``QLinear``), or at load time with ``prepare=True``.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .module import Module

_ST_DTYPES = {
    "F16": (np.uint16, torch.float16), "BF16": (np.uint16, torch.bfloat16), "F32": (np.float32, torch.float32),
    "F64": (np.float64, torch.float64), "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8), "BOOL": (np.uint8, torch.bool),
}
_ST_NAMES = {v[1]: k for k, v in _ST_DTYPES.items()}


def read_safetensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, CPU tensor) for every tensor of a .safetensors file, in file order."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode("utf-8"))
        base = 8 + hlen
        entries = [(k, v) for k, v in header.items() if k != "__metadata__"]
        entries.sort(key=lambda kv: kv[1]["data_offsets"][0])
        for name, meta in entries:
            if meta["dtype"] not in _ST_DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
            npdt, tdt = _ST_DTYPES[meta["dtype"]]
            b, e = meta["data_offsets"]
            f.seek(base + b)
            raw = f.read(e - b)
            shape = tuple(meta["shape"])
            count = int(np.prod(shape)) if shape else 1
            if len(raw) != count * np.dtype(npdt).itemsize:
                raise ValueError(f"{path}: tensor {name} has {len(raw)} bytes for shape {shape} {meta['dtype']}")
            arr = np.frombuffer(raw, dtype=np.dtype(npdt).newbyteorder("<")).astype(npdt, copy=True).reshape(shape)
            t = torch.from_numpy(arr)
            if tdt in (torch.float16, torch.bfloat16):
                t = t.view(tdt)
            elif tdt is torch.bool:
                t = t.to(torch.bool)
            yield name, t


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Write tensors in the safetensors container (used by tests and to re-save sorted act-order layers)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    blobs: List[bytes] = []
    offset = 0
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        if t.dtype not in _ST_NAMES:
            raise ValueError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        if t.dtype in (torch.float16, torch.bfloat16):
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype is torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * ((8 - len(hbytes) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        for raw in blobs:
            f.write(raw)


def _assign(model: Module, name: str, array: torch.Tensor, epilogue, device) -> None:
    """Cast to the buffer's dtype, check the FULL checkpoint shape against the buffer, then hand the tensor to the
    epilogue and store whatever it returns -- the order of the reference (minit/module/checkpoint.py:30-36), whose
    tensor-parallel servers shard inside the epilogue (examples/llama3_70b.py:298-310): the result may be a
    ``CollectiveTensor`` or a torch shard whose shape differs from the declared buffer."""
    spec_shape, spec_dtype = _buffer_spec(model, name)
    from .module import _DTYPES
    array = array.to(_DTYPES[spec_dtype])
    if tuple(array.shape) != tuple(spec_shape):
        raise ValueError(f"{name}: checkpoint shape {tuple(array.shape)} vs buffer {tuple(spec_shape)}")
    value = epilogue(name, array)
    if isinstance(value, torch.Tensor):
        value = value.to(device)
    model.update_buffer(name, value, sharded=not (isinstance(value, torch.Tensor) and tuple(value.shape) == tuple(spec_shape)))


def _buffer_spec(model: Module, name: str):
    if "." in name:
        prefix, suffix = name.split(".", maxsplit=1)
        return _buffer_spec(model.get_child(prefix), suffix)
    if name not in model.buffers:
        raise KeyError(f"{name} is not a buffer of {type(model).__name__}")
    return model.buffers[name]


def load_from_torch(model: Module, path: str, device="cuda") -> Module:
    checkpoint: Dict[str, torch.Tensor] = torch.load(path, map_location="cpu")
    for name, array in checkpoint.items():
        _assign(model, name, array, lambda k, v: v, device)
    return model


def load_from_safetensors(model: Module, paths: Iterable[str], epilogue: Callable[[str, torch.Tensor], torch.Tensor] = lambda k, v: v,
                          device="cuda", prepare: bool = False) -> Module:
    for path in paths:
        for name, array in read_safetensors(path):
            _assign(model, name, array, epilogue, device)
    if prepare:
        prepare_quantized(model)
    return model


def load_from_safetensors_index(model: Module, path: str, epilogue: Callable[[str, torch.Tensor], torch.Tensor] = lambda k, v: v,
                                device="cuda", prepare: bool = False) -> Module:
    with open(path) as f:
        index = json.load(f)
    parts = [os.path.join(os.path.dirname(path), part) for part in dict.fromkeys(index["weight_map"].values())]
    return load_from_safetensors(model, parts, epilogue, device, prepare)


def prepare_quantized(model: Module) -> None:
    """Run the load-time transforms of every quantized layer now (act-order sort, int8 packing) instead of on first use."""
    from .qlinear import QLinear, W8Linear, pack_w8, sort_act_order
    stack = [model]
    while stack:
        mod = stack.pop()
        if isinstance(mod, QLinear) and isinstance(mod.g_idx, torch.Tensor) and mod._groups() is not None and mod._sorted is None:
            try:
                mod._sorted = sort_act_order(mod.qweight, mod.g_idx, mod.scales.shape[0], mod.bits)
            except ValueError:
                mod._sorted = False
        if isinstance(mod, W8Linear) and isinstance(mod.weight, torch.Tensor) and mod._packed is None \
                and mod.weight.shape[0] % 32 == 0 and mod.weight.shape[1] % 8 == 0:
            mod._packed = pack_w8(mod.weight)
        for child in mod.children:
            stack.append(getattr(mod, child))
