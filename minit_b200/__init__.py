"""minit_b200: B200-native (sm_100a) GPTQ int4 / int8 weight-only Linear for MiniT.

Mirrors the call signatures of MiniT's quantized-linear path (minit.quantize,
minit.operator.linalg, minit.functional.linalg, the QLinear modules of
examples/qwen1_5_int8.py, minit.distributed / minit.nccl / minit.collective) on torch CUDA
tensors, with every kernel reached through the C ABI of libminit_b200.so.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is not built)
from .qlinear import (QLinear, QLinearWithBias, W8Linear, pack_w8, quantized_matrix_multiply,
                      quantized_matrix_multiply_noalloc, quantized_matrix_multiply_ordered, sort_act_order, unpack,
                      w8_perchannel_matrix_multiply)
from .feedforward import (QFeedForward, interleave_gate_up, quantized_gate_up_swiglu, quantized_matrix_multiply_residual,
                          swiglu_interleaved)
from .chain import ChainEntry, LinearChain
from .quantize import Dequantize, QuantizedTensor, dequantize
from .operator.linalg import MatrixMultiply
from .functional.linalg import matrix_multiply
from .core.dispatch import dispatch, register_dispatch

__all__ = [
    "QLinear", "QLinearWithBias", "W8Linear", "quantized_matrix_multiply", "quantized_matrix_multiply_noalloc", "w8_perchannel_matrix_multiply",
    "quantized_matrix_multiply_ordered", "sort_act_order", "pack_w8",
    "unpack", "Dequantize", "QuantizedTensor", "dequantize", "MatrixMultiply", "matrix_multiply",
    "dispatch", "register_dispatch",
    "ChainEntry", "LinearChain",
    "QFeedForward", "interleave_gate_up", "quantized_gate_up_swiglu", "quantized_matrix_multiply_residual", "swiglu_interleaved",
]
__version__ = "0.1.0"
