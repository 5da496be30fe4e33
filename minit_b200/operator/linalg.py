"""MatrixMultiply operator record and its implementations.

Reference: minit/operator/linalg.py:9-35 (record + shape rule: the dense right operand is
[N,K], the result [M,N]), minit/quantize/dispatch.py:8-11 (a quantized right operand is
dequantized, then the product is taken), minit/cuda/dispatch.py:59-78 (dense CUDA rule).
Here the quantized rule goes straight to the fused kernel when the operand still carries
its packed tensors.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..core.dispatch import register_dispatch
from ..core.operator import Operator


@dataclass
class MatrixMultiply(Operator):
    ...


def _is_quantized(x, y) -> bool:
    from ..quantize.tensor import QuantizedTensor
    return isinstance(y, QuantizedTensor)


@register_dispatch(MatrixMultiply, predicate=_is_quantized, priority=1)
def _matmul_quantized(op: MatrixMultiply, a: torch.Tensor, b) -> tuple:
    from ..qlinear import quantized_matrix_multiply
    if b.packed is not None:
        qweight, qzeros, bits = b.packed
        return (quantized_matrix_multiply(a, qweight, qzeros, b._scale, b._group, bits=bits),)
    # operands exist only unpacked (one element per byte, what the reference's ``unpack`` produces): four bytes
    # along K are one word of the 8-bit layout (little-endian, examples/qwen1_5_int8.py:40-50 read backwards), so
    # the fused 8-bit kernel takes them after two view-and-copy steps; 4-bit values are 8-bit values below 16.
    # The quantized operand is [K,N] (orientation of the fused kernel, examples/qwen1_5_int8.py:156-200).
    data, zero = b._data, b._zero
    k, n = data.shape
    if data.dtype == torch.uint8 and zero.dtype == torch.uint8 and k % 32 == 0 and n % 8 == 0:
        qweight = data.view(k // 4, 4, n).permute(0, 2, 1).contiguous().view(torch.int32).view(k // 4, n)
        qzeros = zero.contiguous().view(torch.int32)
        return (quantized_matrix_multiply(a, qweight, qzeros, b._scale, b._group, bits=8),)
    w = b.dequantize()          # ragged shapes: dequantize (own kernel), then a plain library GEMM
    return (torch.matmul(a, w),)


@register_dispatch(MatrixMultiply, predicate=lambda x, y: isinstance(y, torch.Tensor))
def _matmul_dense(op: MatrixMultiply, x: torch.Tensor, y: torch.Tensor) -> tuple:
    # dense weights are [out, in] (minit/operator/linalg.py:30-35); plain library GEMM, not part of the quantized path
    if not (x.is_cuda and y.is_cuda):
        raise RuntimeError("minit_b200 operates on CUDA tensors only")
    assert x.dtype == y.dtype
    return (torch.matmul(x, y.t()),)
