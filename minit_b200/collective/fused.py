"""Row-parallel linear with the all-reduce fused into the GEMM kernel (no NCCL on the data path).

The reference turns a row-parallel product into ``Partial`` and all-reduces it with NCCL when it is
consumed (minit/collective/dispatch.py:33-37, minit/collective/tensor.py:72-73).  Here the exchange
happens inside the GEMM epilogue over peer memory: see ``mt_qgemm_allreduce`` in include/minit_b200.h.

The symmetric buffers (one per rank, mapped into every rank's address space) come from
``torch.distributed._symmetric_memory``: torch is the plumbing that allocates and maps them, the
kernel only sees the table of peer pointers.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib
from ..distributed.group import get_world


class FusedAllReduce:
    """Symmetric buffers for the fused row-parallel GEMM: one instance per process group."""

    def __init__(self, group=None, m_max: int = 64, n_max: int = 16384) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        # plain peer loads / stores only: never bind the buffer to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = dist.group.WORLD if group is None else group
        self.nbytes = int(_lib.lib.mt_allreduce_buffer_bytes(m_max, n_max, dist.get_world_size(group)))
        self.m_max, self.n_max = m_max, n_max
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_table = torch.tensor(ptrs, dtype=torch.int64, device=dev)   # device array of peer pointers
        torch.cuda.synchronize()
        dist.barrier(group)   # every rank's buffer is zeroed before anyone's first kernel can raise a flag in it

    @staticmethod
    def check() -> None:
        """Raise ``MinitError`` (``MT_ERR_PEER_TIMEOUT``) if a fused all-reduce since the last check gave up waiting
        for a peer: its output, and everything computed from it, is not valid and differs between ranks.  Reads
        device memory (synchronises): call it where the host waits for the step anyway."""
        _lib.raise_on_error_words()

    def matmul(self, x, qweight, zeros, scales, groups, *, bits: int, bias=None, out=None, flags: int = 0, residual=None):
        """out = sum over ranks of x_r @ W_r (+ bias) (+ residual, the same tensor on every rank), identical on
        every rank, in one kernel per rank."""
        pack = 32 // bits
        *ms, k0 = x.shape
        n0 = qweight.shape[1]
        m = 1
        for d in ms:
            m *= d
        if k0 != qweight.shape[0] * pack or scales.shape[1] != n0 or scales.dtype != x.dtype:
            raise ValueError("shape or dtype mismatch between x, qweight and scales")
        if m > self.m_max or n0 > self.n_max:
            raise ValueError(f"[{m},{n0}] exceeds the symmetric buffer ({self.m_max} x {self.n_max})")
        dev = _lib.require_cuda(x, qweight, zeros, scales, groups, bias, residual)
        if residual is not None and (residual.dtype != x.dtype or residual.numel() != m * n0 or not residual.is_contiguous()):
            raise ValueError("residual must be a contiguous [*ms, N] tensor in x.dtype")
        if out is None:
            out = torch.empty((*ms, n0), dtype=x.dtype, device=dev)
        stream = _lib.current_stream(dev)
        ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, bits))
        with torch.cuda.device(dev):
            rc = _lib.lib.mt_qgemm_residual(stream, x.data_ptr(), qweight.data_ptr(), _lib.ptr(groups), _lib.ptr(zeros),
                                            scales.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), out.data_ptr(), m, n0, k0,
                                            scales.shape[0], bits, _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags,
                                            self.peer_table.data_ptr(), self.rank, self.world, self.nbytes)
        _lib.check(rc, "mt_qgemm_residual")
        return out
