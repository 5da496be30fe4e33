"""Dequantize operator record (reference: minit/quantize/operator.py:5-7) and its CUDA rule
(the reference's rule, minit/quantize/dispatch.py:14-20, runs seven elementwise kernels;
this one is a single bit-exact kernel)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from ..core.dispatch import register_dispatch
from ..core.operator import Operator


@dataclass
class Dequantize(Operator):
    axis: int


@register_dispatch(Dequantize)
def _dequantize(op: Dequantize, data: torch.Tensor, group: torch.Tensor, zero: torch.Tensor, scale: torch.Tensor) -> tuple:
    if op.axis != 0:
        raise ValueError("Dequantize gathers along axis 0 (K), as QuantizedTensor.dequantize does")
    if data.dtype != torch.uint8 or zero.dtype != torch.uint8 or group.dtype != torch.int32:
        raise ValueError("dequantize takes uint8 data / zero (one element per byte) and an int32 group index")
    dev = _lib.require_cuda(data, group, zero, scale)
    k, n = data.shape
    g = scale.shape[0]
    if zero.shape != scale.shape or group.shape != (k,) or scale.shape[1] != n:
        raise ValueError("shape mismatch between data [K,N], group [K], zero [G,N] and scale [G,N]")
    out = torch.empty((k, n), dtype=scale.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_dequant_unpacked(_lib.current_stream(dev), data.data_ptr(), group.data_ptr(), zero.data_ptr(),
                                          scale.data_ptr(), out.data_ptr(), n, k, g, _lib.dtype_code(scale.dtype))
    _lib.check(rc, "mt_dequant_unpacked")
    return (out,)
