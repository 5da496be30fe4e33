"""The gated feed-forward of a decoder layer on quantized linears, with its elementwise steps fused
into the linears.

Reference: ``FeedForward`` (examples/llama3_70b.py:118-130: ``down(silu(gate(x)) * up(x))``;
examples/qwen1_5_int8.py:371-383: ``c_proj(w1(x) * silu(w2(x)))`` on ``QLinearWithBias``) and the
residual add of the decoder block (examples/llama3_70b.py:160-162).  The reference runs the two input
linears, sigmoid, two multiplies and the residual add as separate kernels, each rounding to the
tensor dtype; here the two input linears are ONE linear over interleaved columns whose epilogue
applies silu(gate) * up in fp32, and the residual is added in the epilogue of the output linear.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .module import Module
from .qlinear import QLinear, QLinearWithBias, quantized_matrix_multiply


def interleave_gate_up(gate: Tuple, up: Tuple, *, bits: int = 8):
    """Load-time: two GPTQ linears ``(qweight, qzeros | None, scales, bias | None)`` with the same K, groups
    and N = n_half become one of 2 * n_half columns, blocks of eight = four gate columns then the four up
    columns of the same indices.  Returns ``(qweight, qzeros, scales, bias)``."""
    gq, gz, gs, gb = gate
    uq, uz, us, ub = up
    if gq.shape != uq.shape or gs.shape != us.shape or gq.dtype != torch.int32 or gs.dtype != us.dtype:
        raise ValueError("gate and up must have the same shapes and dtypes")
    if (gz is None) != (uz is None) or (gb is None) != (ub is None):
        raise ValueError("gate and up must both have (or both lack) zeros / bias")
    pack = 32 // bits
    kp, half = gq.shape
    groups = gs.shape[0]
    dev = _lib.require_cuda(gq, uq, gz, uz, gs, us, gb, ub)
    qw = torch.empty((kp, 2 * half), dtype=torch.int32, device=dev)
    sc = torch.empty((groups, 2 * half), dtype=gs.dtype, device=dev)
    qz = torch.empty((groups, 2 * half // pack), dtype=torch.int32, device=dev) if gz is not None else None
    bi = torch.empty((2 * half,), dtype=gb.dtype, device=dev) if gb is not None else None
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_interleave_gate_up(_lib.current_stream(dev), gq.data_ptr(), uq.data_ptr(), _lib.ptr(gz), _lib.ptr(uz),
                                            gs.data_ptr(), us.data_ptr(), _lib.ptr(gb), _lib.ptr(ub),
                                            qw.data_ptr(), _lib.ptr(qz), sc.data_ptr(), _lib.ptr(bi), half, kp * pack, groups, bits)
    _lib.check(rc, "mt_interleave_gate_up")
    return qw, qz, sc, bi


def swiglu_interleaved(y: torch.Tensor) -> torch.Tensor:
    """out[.., 4b + j] = silu(y[.., 8b + j]) * y[.., 8b + 4 + j] for j < 4: the activation on the interleaved layout."""
    dev = _lib.require_cuda(y)
    *ms, n0 = y.shape
    m = y.numel() // max(n0, 1)
    out = torch.empty((*ms, n0 // 2), dtype=y.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_swiglu(_lib.current_stream(dev), y.data_ptr(), out.data_ptr(), m, n0, _lib.dtype_code(y.dtype))
    _lib.check(rc, "mt_swiglu")
    return out


def quantized_gate_up_swiglu(x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor], scales: torch.Tensor, *,
                             bits: int = 8, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                             flags: int = 0) -> torch.Tensor:
    """out[*ms, N/2] = silu(gate(x)) * up(x) for a linear prepared with ``interleave_gate_up`` (one kernel at M <= 2)."""
    pack = 32 // bits
    *ms, k0 = x.shape
    n0 = qweight.shape[1]
    if k0 != qweight.shape[0] * pack or scales.shape[1] != n0 or scales.dtype != x.dtype:
        raise ValueError("shape or dtype mismatch between x, qweight and scales")
    dev = _lib.require_cuda(x, qweight, zeros, scales, bias)
    m = 1
    for d in ms:
        m *= d
    if out is None:
        out = torch.empty((*ms, n0 // 2), dtype=x.dtype, device=dev)
    # the GEMV has the epilogue at M <= 2 (N % 128 == 0, group size % 32 == 0); otherwise the GEMM writes a scratch row first
    scratch = torch.empty((m, n0), dtype=x.dtype, device=dev) if (m > 2 or n0 % 128 or (k0 // scales.shape[0]) % 32) else None
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, bits))
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm_swiglu(stream, x.data_ptr(), qweight.data_ptr(), _lib.ptr(zeros), scales.data_ptr(), _lib.ptr(bias),
                                      out.data_ptr(), _lib.ptr(scratch), m, n0, k0, scales.shape[0], bits,
                                      _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags)
    _lib.check(rc, "mt_qgemm_swiglu")
    return out


def quantized_matrix_multiply_residual(x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor], scales: torch.Tensor,
                                       groups: Optional[torch.Tensor], residual: torch.Tensor, *, bits: int = 8,
                                       bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                                       flags: int = 0) -> torch.Tensor:
    """out = residual + (x @ W (+ bias)) on one GPU (the tensor-parallel form is ``FusedAllReduce.matmul(residual=)``)."""
    pack = 32 // bits
    *ms, k0 = x.shape
    n0 = qweight.shape[1]
    if k0 != qweight.shape[0] * pack or scales.shape[1] != n0 or scales.dtype != x.dtype:
        raise ValueError("shape or dtype mismatch between x, qweight and scales")
    m = 1
    for d in ms:
        m *= d
    if residual.dtype != x.dtype or residual.numel() != m * n0 or not residual.is_contiguous():
        raise ValueError("residual must be a contiguous [*ms, N] tensor in x.dtype")
    dev = _lib.require_cuda(x, qweight, zeros, scales, groups, bias, residual)
    if out is None:
        out = torch.empty((*ms, n0), dtype=x.dtype, device=dev)
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, bits))
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm_residual(stream, x.data_ptr(), qweight.data_ptr(), _lib.ptr(groups), _lib.ptr(zeros), scales.data_ptr(),
                                        _lib.ptr(bias), residual.data_ptr(), out.data_ptr(), m, n0, k0, scales.shape[0], bits,
                                        _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags, None, 0, 1, 0)
    _lib.check(rc, "mt_qgemm_residual")
    return out


class QFeedForward(Module):
    """``FeedForward(hidden_size, internal_size)`` of the reference on GPTQ linears.  The three linears
    keep the reference's buffers and names (so checkpoints load unchanged); on first use gate and up are
    interleaved into one linear (a second copy of their weights).  ``names`` = (gate, up, down):
    ("gate_proj", "up_proj", "down_proj") for Llama / Mistral, ("w2", "w1", "c_proj") for Qwen, whose
    ``w2`` is the activated branch."""

    def __init__(self, hidden_size: int, internal_size: int, nr_groups_in: int, nr_groups_out: int, bits: int = 8,
                 bias: bool = False, names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj"),
                 dtype: str = "float16") -> None:
        super().__init__()
        cls = QLinearWithBias if bias else QLinear
        self.bits = bits
        self.gate = self.register_module(names[0], cls(hidden_size, internal_size, nr_groups_in, bits, dtype))
        self.up = self.register_module(names[1], cls(hidden_size, internal_size, nr_groups_in, bits, dtype))
        self.down = self.register_module(names[2], cls(internal_size, hidden_size, nr_groups_out, bits, dtype))
        for name, child in zip(names, (self.gate, self.up, self.down)):
            setattr(self, name, child)                       # children are looked up by their registered names
        self._fused = None

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        super().update_buffer(name, value, sharded)
        self._fused = None                                   # the interleaved copy is rebuilt on the next call

    def _gate_up(self):
        if self._fused is None:
            for lin in (self.gate, self.up):
                if lin._groups() is not None:
                    raise ValueError("act-order gate / up projections are not fused: call the three linears separately")
            gb = getattr(self.gate, "bias", None)
            ub = getattr(self.up, "bias", None)
            self._fused = interleave_gate_up((self.gate.qweight, self.gate.qzeros, self.gate.scales, gb),
                                             (self.up.qweight, self.up.qzeros, self.up.scales, ub), bits=self.bits)
        return self._fused

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        qw, qz, sc, bi = self._gate_up()
        h = quantized_gate_up_swiglu(x, qw, qz, sc, bits=self.bits, bias=bi)
        db = getattr(self.down, "bias", None)
        if residual is None:
            return self.down._matmul(h, db)
        groups = self.down._groups()
        return quantized_matrix_multiply_residual(h, self.down.qweight, self.down.qzeros, self.down.scales, groups, residual,
                                                  bits=self.bits, bias=db)
