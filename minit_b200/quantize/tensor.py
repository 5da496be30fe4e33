"""QuantizedTensor(data, group, zero, scale) (reference: minit/quantize/tensor.py:9-30).

``data`` [K,N] and ``zero`` [G,N] hold one element per uint8, ``group`` [K] int32 maps k to
its group, ``scale`` [G,N] is fp16/bf16.  ``packed`` optionally keeps the int32-packed
originals (qweight, qzeros, bits) so a matrix product can use the fused kernel instead of
dequantize-then-matmul.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from .functional import dequantize


def _torch(x):
    view = getattr(x, "as_torch", None)
    return view() if callable(view) else x


class QuantizedTensor:
    def __init__(self, data: torch.Tensor, group: torch.Tensor, zero: torch.Tensor, scale: torch.Tensor,
                 packed: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None) -> None:
        # operands may arrive in the compat layer's device-tensor wrapper (``minit_b200.compat.tensor.CUDATensor``)
        self._data = _torch(data)
        self._group = _torch(group)
        self._zero = _torch(zero)
        self._scale = _torch(scale)
        self.packed = packed

    @property
    def shape(self):
        return self._data.shape

    @property
    def dtype(self):
        return f"q{str(self._data.dtype).replace('torch.', '')}"

    @property
    def device(self):
        return self._data.device

    def type(self):
        return type(self)

    def dequantize(self) -> torch.Tensor:
        if self.packed is not None:
            qweight, qzeros, bits = self.packed
            return dequantize_packed(qweight, self._group, qzeros, self._scale, bits)
        return dequantize(self._data, self._group, self._zero, self._scale, 0)


def dequantize_packed(qweight: torch.Tensor, g_idx: Optional[torch.Tensor], qzeros: Optional[torch.Tensor],
                      scales: torch.Tensor, bits: int) -> torch.Tensor:
    """W[K,N] straight from the packed GPTQ tensors (one kernel, bit-exact with the reference formula)."""
    dev = _lib.require_cuda(qweight, g_idx, qzeros, scales)
    pack = 32 // bits
    k, n = qweight.shape[0] * pack, qweight.shape[1]
    out = torch.empty((k, n), dtype=scales.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_dequant(_lib.current_stream(dev), qweight.data_ptr(), _lib.ptr(g_idx), _lib.ptr(qzeros),
                                 scales.data_ptr(), out.data_ptr(), n, k, scales.shape[0], bits, _lib.dtype_code(scales.dtype))
    _lib.check(rc, "mt_dequant")
    return out
