"""Several decode linears of a layer in one launch (``mt_qgemm_chain``).

The reference issues one launch of its fused kernel per linear (examples/qwen1_5_int8.py:244-267) and, under tensor
parallelism, an all_reduce after every row-parallel one (minit/nccl/kernel.py:51-53).  At one or two tokens those
launches are so short that the boundaries between them cost as much as the streaming of the weights, so a
``LinearChain`` hands the whole list to one resident kernel: entries run in order, an entry may read what an earlier
one wrote, and the weight stream does not stop between them.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from .qlinear import _validate_gptq_call


class ChainEntry:
    """One linear of a chain: out = x @ W (+ bias) (+ all-reduce) (+ residual), or SwiGLU of interleaved gate/up
    columns (``epilogue='swiglu'``, out is [.., N/2]).  The tensors are used in place at every call of the chain."""

    def __init__(self, x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor], scales: torch.Tensor,
                 out: torch.Tensor, *, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 epilogue: Optional[str] = None, allreduce: bool = False) -> None:
        if epilogue not in (None, "swiglu"):
            raise ValueError("epilogue must be None or 'swiglu'")
        self.x, self.qweight, self.zeros, self.scales, self.out = x, qweight, zeros, scales, out
        self.bias, self.residual, self.epilogue, self.allreduce = bias, residual, epilogue, bool(allreduce)


class LinearChain:
    """A fixed list of at most ``_lib.CHAIN_MAX`` decode linears (M <= 2), launched together by ``__call__``.

    ``fused`` is the ``FusedAllReduce`` whose symmetric buffers the entries with ``allreduce=True`` exchange through
    (required when any entry has it and the group has more than one rank).  When the library answers that the list
    does not fit one launch, ``__call__`` issues the same linears one by one through the same C ABI.
    """

    def __init__(self, entries: Sequence[ChainEntry], *, bits: int, fused=None, flags: int = 0) -> None:
        if not entries:
            raise ValueError("a chain needs at least one entry")
        self.entries = list(entries)
        self.bits, self.flags, self.fused = bits, flags, fused
        self.m = None
        dev = None
        dtype = self.entries[0].x.dtype
        arr = (_lib.ChainLinear * len(self.entries))()
        max_bytes = 0
        for i, e in enumerate(self.entries):
            ms, m, k0, n0, g1 = _validate_gptq_call(e.x, e.qweight, e.zeros, e.scales, None, e.bias, bits)
            d = _lib.require_cuda(e.x, e.qweight, e.zeros, e.scales, e.bias, e.residual, e.out)
            if dev is None:
                dev, self.m = d, m
            if d != dev or m != self.m or e.x.dtype != dtype:
                raise ValueError("all entries of a chain share the device, the row count and the dtype")
            n_out = n0 // 2 if e.epilogue == "swiglu" else n0
            if e.out.dtype != dtype or e.out.numel() != m * n_out or not e.out.is_contiguous() or not e.x.is_contiguous():
                raise ValueError(f"entry {i}: out must be a contiguous [{m},{n_out}] tensor in x.dtype and x contiguous")
            if e.residual is not None and (e.residual.dtype != dtype or e.residual.numel() != m * n0 or not e.residual.is_contiguous()):
                raise ValueError(f"entry {i}: residual must be a contiguous [{m},{n0}] tensor in x.dtype")
            if e.allreduce and fused is not None and (m > fused.m_max or n0 > fused.n_max):
                raise ValueError(f"entry {i}: [{m},{n0}] exceeds the symmetric buffer ({fused.m_max} x {fused.n_max})")
            arr[i] = _lib.ChainLinear(e.x.data_ptr(), e.qweight.data_ptr(), _lib.ptr(e.zeros), e.scales.data_ptr(), _lib.ptr(e.bias),
                                      _lib.ptr(e.residual), e.out.data_ptr(), n0, k0, g1,
                                      _lib.EPILOGUE_SWIGLU if e.epilogue == "swiglu" else _lib.EPILOGUE_NONE, int(e.allreduce))
            max_bytes = max(max_bytes, int(_lib.lib.mt_workspace_bytes(m, n0, k0, bits)))
        world = fused.world if fused is not None else 1
        if any(e.allreduce for e in self.entries) and fused is None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                raise ValueError("entries with allreduce=True need the FusedAllReduce of the group")
        self._arr, self._dev, self._dtype, self._ws_bytes, self._world = arr, dev, dtype, max_bytes, world
        self.single_launch = None   # set by the first call: whether the list runs as one launch

    def __call__(self) -> None:
        dev = self._dev
        stream = _lib.current_stream(dev)
        ws = _lib.workspace(dev, stream, self._ws_bytes)
        f = self.fused
        with torch.cuda.device(dev):
            rc = _lib.lib.mt_qgemm_chain(stream, ctypes.addressof(self._arr), len(self.entries), self.m, self.bits,
                                         _lib.dtype_code(self._dtype), ws.data_ptr(), ws.numel(), self.flags,
                                         f.peer_table.data_ptr() if f is not None else None,
                                         f.rank if f is not None else 0, self._world, f.nbytes if f is not None else 0)
        if rc == _lib.ERR_UNSUPPORTED:
            self.single_launch = False
            self._one_by_one()
            return
        _lib.check(rc, "mt_qgemm_chain")
        self.single_launch = True

    def _one_by_one(self) -> None:
        from .feedforward import quantized_gate_up_swiglu, quantized_matrix_multiply_residual
        from .qlinear import quantized_matrix_multiply
        for e in self.entries:
            if e.epilogue == "swiglu":
                quantized_gate_up_swiglu(e.x, e.qweight, e.zeros, e.scales, bits=self.bits, bias=e.bias, out=e.out, flags=self.flags)
            elif e.allreduce and self.fused is not None and self._world > 1:
                self.fused.matmul(e.x, e.qweight, e.zeros, e.scales, None, bits=self.bits, bias=e.bias, out=e.out,
                                  flags=self.flags, residual=e.residual)
            elif e.residual is not None:
                quantized_matrix_multiply_residual(e.x, e.qweight, e.zeros, e.scales, None, e.residual, bits=self.bits,
                                                   bias=e.bias, out=e.out, flags=self.flags)
            else:
                quantized_matrix_multiply(e.x, e.qweight, e.zeros, e.scales, None, bits=self.bits, bias=e.bias, out=e.out,
                                          flags=self.flags)
