"""The quantized-linear operators with the reference's Python call signatures.

Reference (examples/qwen1_5_int8.py): ``unpack`` :40-50, ``quantized_matrix_multiply`` :244-267,
``QLinear`` :270-289, ``QLinearWithBias`` :292-317.  Tensors are torch CUDA tensors; every
function is one call into the C ABI on the current stream (no per-call allocation besides
the output, no synchronisation).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .module import Module
from .quantize.tensor import QuantizedTensor

default_dtype = "float16"


def unpack(x: torch.Tensor, axis: int, bits: int = 8) -> torch.Tensor:
    """int32-packed [.., ..] -> one element per uint8 along ``axis`` (little-endian inside the word)."""
    if x.dtype != torch.int32 or x.dim() != 2:
        raise ValueError("unpack takes a 2-D int32 tensor")
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1")
    dev = _lib.require_cuda(x)
    pack = 32 // bits
    rows = x.shape[0] * pack if axis == 0 else x.shape[0]
    cols = x.shape[1] if axis == 0 else x.shape[1] * pack
    out = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_unpack(_lib.current_stream(dev), x.data_ptr(), out.data_ptr(), rows, cols, bits, axis)
    _lib.check(rc, "mt_unpack")
    return out


def _validate_gptq_call(x, qweight, zeros, scales, groups, bias, bits: int):
    """Shape and dtype contract shared by every wrapper of the fused kernel (examples/qwen1_5_int8.py:247-254, plus the
    integer dtypes the kernels index with): raises ValueError before anything reaches the C call.  Returns (ms, m, k, n, g)."""
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    pack = 32 // bits
    *ms, k0 = x.shape
    if qweight.dim() != 2 or scales.dim() != 2:
        raise ValueError("qweight and scales must be 2-D")
    pk1, n0 = qweight.shape
    g1, n2 = scales.shape
    if not (k0 == pk1 * pack and n0 == n2):
        raise ValueError(f"shape mismatch: x[..,{k0}] qweight[{pk1}*{pack},{n0}] scales[{g1},{n2}]")
    if qweight.dtype != torch.int32:
        raise ValueError("qweight must be int32 (packed words)")
    if zeros is not None and (tuple(zeros.shape) != (g1, n0 // pack) or zeros.dtype != torch.int32):
        raise ValueError(f"zeros must be int32 [{g1},{n0 // pack}], got {zeros.dtype} {tuple(zeros.shape)}")
    if groups is not None and (tuple(groups.shape) != (k0,) or groups.dtype != torch.int32):
        raise ValueError(f"groups must be int32 [{k0}], got {groups.dtype} {tuple(groups.shape)}")
    if scales.dtype != x.dtype:
        raise ValueError("scales.dtype must equal x.dtype")
    if bias is not None and (bias.dtype != x.dtype or tuple(bias.shape) != (n0,)):
        raise ValueError("bias must be [N] in x.dtype")
    m = 1
    for d in ms:
        m *= d
    return ms, m, k0, n0, g1


def quantized_matrix_multiply(x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor],
                              scales: torch.Tensor, groups: Optional[torch.Tensor], *, bits: int = 8,
                              bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                              flags: int = 0) -> torch.Tensor:
    """out[*ms, N] = x[*ms, K] @ W[K, N] (+ bias) with W = (q - (z + 1)) * s per group.

    Same positional arguments as the reference (x, qweight, zeros, scales, groups); ``bits``
    defaults to 8 because that is the only width the reference instantiates.  ``groups`` is
    the per-k group index (g_idx) or None for contiguous groups; ``zeros`` None means the
    symmetric midpoint.  The shape contract is the reference's (examples/qwen1_5_int8.py:247-254).
    """
    ms, m, k0, n0, g1 = _validate_gptq_call(x, qweight, zeros, scales, groups, bias, bits)
    dev = _lib.require_cuda(x, qweight, zeros, scales, groups, bias)
    if out is None:
        out = torch.empty((*ms, n0), dtype=x.dtype, device=dev)
    else:
        _lib.require_cuda(out)
        if tuple(out.shape) != (*ms, n0) or out.dtype != x.dtype:
            raise ValueError("out has the wrong shape or dtype")
    stream = _lib.current_stream(dev)
    need = _lib.lib.mt_workspace_bytes(m, n0, k0, bits)
    ws = _lib.workspace(dev, stream, need)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm(stream, x.data_ptr(), qweight.data_ptr(), _lib.ptr(groups), _lib.ptr(zeros),
                               scales.data_ptr(), _lib.ptr(bias), out.data_ptr(), m, n0, k0, g1, bits,
                               _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags)
    _lib.check(rc, "mt_qgemm")
    return out


def sort_act_order(qweight: torch.Tensor, g_idx: torch.Tensor, nr_groups: int, bits: int = 8):
    """Load-time preparation of an act-order (desc_act) GPTQ layer: sort the rows of ``qweight`` by group
    (stable), so that the contiguous-group kernels apply, and return ``(qweight_sorted, perm)``;
    ``x[..., perm] @ W_sorted == x @ W``.  Raises when ``g_idx`` does not assign exactly K / nr_groups rows
    to every group (such a layer stays on the g_idx kernel).  One device->host read of a status word."""
    pack = 32 // bits
    k0 = qweight.shape[0] * pack
    if tuple(g_idx.shape) != (k0,) or g_idx.dtype != torch.int32 or qweight.dtype != torch.int32:
        raise ValueError("qweight int32 [K/pack,N] and g_idx int32 [K] expected")
    dev = _lib.require_cuda(qweight, g_idx)
    perm = torch.empty(k0, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty_like(qweight)
    with torch.cuda.device(dev):
        stream = _lib.current_stream(dev)
        _lib.check(_lib.lib.mt_act_order_perm(stream, g_idx.data_ptr(), perm.data_ptr(), status.data_ptr(), k0, nr_groups),
                   "mt_act_order_perm")
        st = int(status.item())
        if st != 0:
            raise ValueError("g_idx is not a permutation of equal-sized groups" if st == 1 else "g_idx holds a group index out of range")
        _lib.check(_lib.lib.mt_repack_rows(stream, qweight.data_ptr(), perm.data_ptr(), out.data_ptr(), qweight.shape[1], k0, bits),
                   "mt_repack_rows")
    return out, perm


def quantized_matrix_multiply_ordered(x: torch.Tensor, qweight_sorted: torch.Tensor, zeros: Optional[torch.Tensor],
                                      scales: torch.Tensor, perm: torch.Tensor, *, bits: int = 8,
                                      bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                                      flags: int = 0) -> torch.Tensor:
    """``quantized_matrix_multiply`` for a layer prepared with ``sort_act_order``: out = x[..., perm] @ W_sorted.
    At M <= 2 the gather is part of the GEMV; for larger M one extra launch gathers x into a scratch tensor."""
    pack = 32 // bits
    *ms, k0 = x.shape
    pk1, n0 = qweight_sorted.shape
    g1 = scales.shape[0]
    if k0 != pk1 * pack or scales.shape[1] != n0 or scales.dtype != x.dtype or tuple(perm.shape) != (k0,) or perm.dtype != torch.int32:
        raise ValueError("shape or dtype mismatch between x, qweight, scales and perm")
    dev = _lib.require_cuda(x, qweight_sorted, zeros, scales, perm, bias)
    m = 1
    for d in ms:
        m *= d
    if out is None:
        out = torch.empty((*ms, n0), dtype=x.dtype, device=dev)
    scratch = torch.empty((m, k0), dtype=x.dtype, device=dev) if m > 2 else None
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, bits))
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm_ordered(stream, x.data_ptr(), perm.data_ptr(), _lib.ptr(scratch), qweight_sorted.data_ptr(),
                                       _lib.ptr(zeros), scales.data_ptr(), _lib.ptr(bias), out.data_ptr(), m, n0, k0, g1, bits,
                                       _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags)
    _lib.check(rc, "mt_qgemm_ordered")
    return out


def pack_w8(weight: torch.Tensor) -> torch.Tensor:
    """Load-time: plain int8 weights [K,N] -> the 8-bit GPTQ word layout int32 [K/4,N] (stored value w + 128)."""
    if weight.dtype != torch.int8 or weight.dim() != 2 or weight.shape[0] % 4 or weight.shape[1] % 4:
        raise ValueError("weight must be int8 [K,N] with K and N multiples of 4")
    dev = _lib.require_cuda(weight)
    out = torch.empty((weight.shape[0] // 4, weight.shape[1]), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.mt_w8_pack(_lib.current_stream(dev), weight.data_ptr(), out.data_ptr(), weight.shape[1], weight.shape[0]),
                   "mt_w8_pack")
    return out


def quantized_matrix_multiply_noalloc(x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor],
                                      scales: torch.Tensor, groups: Optional[torch.Tensor], out: torch.Tensor, *,
                                      bits: int = 8, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``quantized_matrix_multiply`` for programs that must not allocate device memory while
    they run -- a server that handed the whole GPU to its own pool, or a decode loop that cannot
    absorb an allocator's synchronisation.  The caller supplies ``out``; the scratch the kernel
    needs lives in a fixed 8 MiB array inside the library, so neither this function nor the C
    call under it allocates.  Shapes whose scratch would not fit raise (status -10); calls share
    the array, so do not let two of them overlap on the GPU.  Call it once before any stream
    capture on a device: the first call looks up the array's address."""
    ms, m, k0, n0, _ = _validate_gptq_call(x, qweight, zeros, scales, groups, bias, bits)
    if tuple(out.shape) != (*ms, n0) or out.dtype != x.dtype:
        raise ValueError("out has the wrong shape or dtype")
    dev = _lib.require_cuda(x, qweight, zeros, scales, groups, bias, out)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm_static(_lib.current_stream(dev), x.data_ptr(), qweight.data_ptr(), _lib.ptr(groups),
                                      _lib.ptr(zeros), scales.data_ptr(), _lib.ptr(bias), out.data_ptr(), m, n0, k0,
                                      scales.shape[0], bits, _lib.dtype_code(x.dtype), 0)
    _lib.check(rc, "mt_qgemm_static")
    return out


def w8_perchannel_matrix_multiply(x: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor, *,
                                  bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                                  flags: int = 0) -> torch.Tensor:
    """out = (x @ float(weight)) * scales (+ bias); weight int8 [K,N], scales [N] in x.dtype."""
    *ms, k0 = x.shape
    if weight.dtype != torch.int8 or weight.dim() != 2 or weight.shape[0] != k0:
        raise ValueError("weight must be int8 [K,N]")
    n0 = weight.shape[1]
    if tuple(scales.shape) != (n0,) or scales.dtype != x.dtype:
        raise ValueError("scales must be [N] in x.dtype")
    if bias is not None and (bias.dtype != x.dtype or tuple(bias.shape) != (n0,)):
        raise ValueError("bias must be [N] in x.dtype")
    dev = _lib.require_cuda(x, weight, scales, bias)
    m = 1
    for d in ms:
        m *= d
    if out is None:
        out = torch.empty((*ms, n0), dtype=x.dtype, device=dev)
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, 8))
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_w8_perchannel_gemm(stream, x.data_ptr(), weight.data_ptr(), scales.data_ptr(), _lib.ptr(bias),
                                            out.data_ptr(), m, n0, k0, _lib.dtype_code(x.dtype), ws.data_ptr(), ws.numel(), flags)
    _lib.check(rc, "mt_w8_perchannel_gemm")
    return out


def _trivial_groups(g_idx: torch.Tensor, nr_groups: int) -> bool:
    k = g_idx.numel()
    if k % nr_groups:
        return False
    ref = torch.arange(k, device=g_idx.device, dtype=torch.int32) // (k // nr_groups)
    return bool(torch.equal(g_idx, ref))


class QLinear(Module):
    """GPTQ linear: buffers qweight (in/pack, out) int32, qzeros (nr_groups, out/pack) int32,
    scales (nr_groups, out), g_idx (in,) int32.  ``bits`` = 8 reproduces the reference module;
    4 is the int4 layout."""

    def __init__(self, in_features: int, out_features: int, nr_groups: int, bits: int = 8,
                 dtype: str = default_dtype) -> None:
        super().__init__()
        pack = 32 // bits
        self.bits = bits
        self.qweight = self.register_buffer("qweight", (in_features // pack, out_features), "int32")
        self.qzeros = self.register_buffer("qzeros", (nr_groups, out_features // pack), "int32")
        self.scales = self.register_buffer("scales", (nr_groups, out_features), dtype)
        self.g_idx = self.register_buffer("g_idx", (in_features,), "int32")
        self._groups_arg = "unchecked"
        self._sorted = None       # (qweight_sorted, perm) of an act-order layer, built on first use

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        super().update_buffer(name, value, sharded)
        if name in ("g_idx", "qweight"):
            self._groups_arg = "unchecked"
            self._sorted = None

    def _groups(self):
        # a g_idx that is just k // group_size selects the faster contiguous-group kernel;
        # decided once per load (one device->host read), not per call
        if self._groups_arg == "unchecked":
            self._groups_arg = None if _trivial_groups(self.g_idx, self.scales.shape[0]) else self.g_idx
        return self._groups_arg

    @property
    def weight(self) -> QuantizedTensor:
        return QuantizedTensor(unpack(self.qweight, 0, self.bits), self.g_idx, unpack(self.qzeros, 1, self.bits),
                               self.scales, packed=(self.qweight, self.qzeros, self.bits))

    def _matmul(self, x: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        groups = self._groups()
        if groups is None:
            return quantized_matrix_multiply(x, self.qweight, self.qzeros, self.scales, None, bits=self.bits, bias=bias)
        # act-order: sort the rows by group once (a second copy of qweight), then every call is a contiguous-group
        # kernel reading x through the permutation; a g_idx with unequal groups keeps the per-k lookup kernel
        if self._sorted is None:
            try:
                self._sorted = sort_act_order(self.qweight, self.g_idx, self.scales.shape[0], self.bits)
            except ValueError:
                self._sorted = False
        if self._sorted is False:
            return quantized_matrix_multiply(x, self.qweight, self.qzeros, self.scales, groups, bits=self.bits, bias=bias)
        qw, perm = self._sorted
        return quantized_matrix_multiply_ordered(x, qw, self.qzeros, self.scales, perm, bits=self.bits, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._matmul(x, None)


class QLinearWithBias(QLinear):
    def __init__(self, in_features: int, out_features: int, nr_groups: int, bits: int = 8,
                 dtype: str = default_dtype) -> None:
        super().__init__(in_features, out_features, nr_groups, bits, dtype)
        self.bias = self.register_buffer("bias", (out_features,), dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # the reference adds the bias with two extra kernels (examples/qwen1_5_int8.py:313-316); here it is the GEMM epilogue
        return self._matmul(x, self.bias)


class W8Linear(Module):
    """int8 weight-only linear with one scale per output channel: weight (in, out) int8, scales (out,)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype: str = default_dtype) -> None:
        super().__init__()
        self.weight = self.register_buffer("weight", (in_features, out_features), "int8")
        self.scales = self.register_buffer("scales", (out_features,), dtype)
        self.bias = self.register_buffer("bias", (out_features,), dtype) if bias else None
        self._packed = None       # the weights in the GPTQ word layout, built on first use

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        super().update_buffer(name, value, sharded)
        if name == "weight":
            self._packed = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # packed once into the 8-bit GPTQ layout (one group, stored zero 127) the layer runs on the GPTQ kernels:
        # CUDA-core GEMV at M <= 2, tcgen05 at M > 64
        k0, n0 = self.weight.shape
        if k0 % 32 or n0 % 8:
            return w8_perchannel_matrix_multiply(x, self.weight, self.scales, bias=self.bias)
        if self._packed is None:
            self._packed = pack_w8(self.weight)
        return quantized_matrix_multiply(x, self._packed, None, self.scales.view(1, -1), None, bits=8, bias=self.bias)
