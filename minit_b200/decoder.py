"""The decoder layer around the quantized linears, for decode-sized batches of one sequence.

Reference (examples/llama3_70b.py): ``RMSNorm`` :133-141, ``Attention`` :58-115, ``TransformerBlock``
:144-162, rotary tables :206-212.  Differences a caller must know: the KV cache is preallocated
(``KVCache(capacity, ...)``) and appended in place instead of growing by ``F.tie``; it stores each kv head
once, not ``nr_groups`` times; q, k and v come from ONE linear over the concatenated columns; the
residual adds are folded into the output linears.  Every step is one call into the C ABI.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .feedforward import QFeedForward, quantized_matrix_multiply_residual
from .module import Module
from .qlinear import QLinear, QLinearWithBias, quantized_matrix_multiply


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.rms_norm(x, weight, axis=-1, eps)`` (minit/functional/special.py:11-16)."""
    dev = _lib.require_cuda(x, weight)
    h = x.shape[-1]
    if weight.shape != (h,) or weight.dtype != x.dtype or not x.is_contiguous():
        raise ValueError("weight must be [H] in x.dtype and x contiguous")
    rows = x.numel() // max(h, 1)
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_rms_norm(_lib.current_stream(dev), x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, h, eps,
                                  _lib.dtype_code(x.dtype))
    _lib.check(rc, "mt_rms_norm")
    return out


def rope_tables(head_size: int, size: int, theta: float = 5e5, dtype: torch.dtype = torch.float16, device="cuda"):
    """cos / sin of position * theta^(-2i/d), rounded to ``dtype`` as the reference stores them
    (examples/llama3_70b.py:206-212) and kept as fp32 for the kernel."""
    freqs = (1.0 / theta) ** (torch.arange(0, head_size // 2, dtype=torch.float32) * (2.0 / head_size))
    ang = torch.arange(0, size, dtype=torch.float32)[:, None] * freqs[None, :]
    return (ang.cos().to(dtype).float().to(device).contiguous(), ang.sin().to(dtype).float().to(device).contiguous())


class KVCache:
    """Preallocated cache of one layer: k, v [capacity, kv_heads, head_size]; ``length`` rows are valid."""

    def __init__(self, capacity: int, kv_heads: int, head_size: int, dtype: torch.dtype = torch.float16, device="cuda") -> None:
        self.k = torch.zeros((capacity, kv_heads, head_size), dtype=dtype, device=device)
        self.v = torch.zeros((capacity, kv_heads, head_size), dtype=dtype, device=device)
        self.capacity, self.kv_heads, self.head_size = capacity, kv_heads, head_size
        self.length = 0


def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, cache: KVCache, nr_querys: int, offset: int,
                offset_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate the q and k heads of fused qkv rows [M, (hq + 2 hkv) d] and append k, v to the cache at rows
    offset .. offset + M - 1; returns q [M, hq, d]."""
    dev = _lib.require_cuda(qkv, cos, sin, cache.k, cache.v, offset_dev)
    m = qkv.shape[0]
    hkv, d = cache.kv_heads, cache.head_size
    if qkv.shape != (m, (nr_querys + 2 * hkv) * d) or not qkv.is_contiguous() or cos.dtype != torch.float32 or cos.shape != sin.shape:
        raise ValueError("qkv must be [M, (hq + 2 hkv) d] contiguous and the tables fp32 of one shape")
    q = torch.empty((m, nr_querys, d), dtype=qkv.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_rope_append(_lib.current_stream(dev), qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(),
                                     cache.k.data_ptr(), cache.v.data_ptr(), m, nr_querys, hkv, d, offset, _lib.ptr(offset_dev),
                                     cache.capacity, cos.shape[0], _lib.dtype_code(qkv.dtype))
    _lib.check(rc, "mt_rope_append")
    return q


def qkv_rope_append(x: torch.Tensor, qweight: torch.Tensor, zeros: Optional[torch.Tensor], scales: torch.Tensor,
                    cos: torch.Tensor, sin: torch.Tensor, cache: KVCache, nr_querys: int, offset: int, *, bits: int = 8,
                    bias: Optional[torch.Tensor] = None, offset_dev: Optional[torch.Tensor] = None, flags: int = 0) -> torch.Tensor:
    """The fused q/k/v linear with the rotary embedding and the cache append as its epilogue (one kernel at M <= 2):
    returns q [M, hq, d]; k and v of the M tokens land in the cache at rows offset .. offset + M - 1."""
    dev = _lib.require_cuda(x, qweight, zeros, scales, cos, sin, cache.k, cache.v, bias, offset_dev)
    pack = 32 // bits
    m, k0 = x.shape
    hkv, d = cache.kv_heads, cache.head_size
    n0 = (nr_querys + 2 * hkv) * d
    if qweight.shape != (k0 // pack, n0) or scales.shape[1] != n0 or scales.dtype != x.dtype or cos.dtype != torch.float32:
        raise ValueError("shape or dtype mismatch between x, qweight, scales and the tables")
    q = torch.empty((m, nr_querys, d), dtype=x.dtype, device=dev)
    scratch = torch.empty((m, n0), dtype=x.dtype, device=dev) if (m > 2 or d != 128 or (k0 // scales.shape[0]) % 32) else None
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, _lib.lib.mt_workspace_bytes(m, n0, k0, bits))
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_qgemm_rope_append(stream, x.data_ptr(), qweight.data_ptr(), _lib.ptr(zeros), scales.data_ptr(), _lib.ptr(bias),
                                           cos.data_ptr(), sin.data_ptr(), q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                           _lib.ptr(scratch), m, nr_querys, hkv, d, k0, scales.shape[0], bits, _lib.dtype_code(x.dtype),
                                           offset, _lib.ptr(offset_dev), cache.capacity, cos.shape[0], ws.data_ptr(), ws.numel(), flags)
    _lib.check(rc, "mt_qgemm_rope_append")
    return q


_att_ws = {}


def attention_decode(q: torch.Tensor, cache: KVCache, offset: int, offset_dev: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(q k^T / sqrt(d) + causal mask) v for M new tokens (q [M, hq, d]) at positions offset .. against the
    cache rows 0 .. offset + token; returns [M, hq * d]."""
    dev = _lib.require_cuda(q, cache.k, cache.v, offset_dev)
    m, hq, d = q.shape
    max_len = cache.capacity if offset_dev is not None else offset + m
    need = _lib.lib.mt_attention_workspace_bytes(m, cache.kv_heads, max_len)
    stream = _lib.current_stream(dev)
    key = (dev.index, stream)
    ws = _att_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)       # zeroed once; the kernel leaves it zeroed
        _att_ws[key] = ws
    if out is None:
        out = torch.empty((m, hq * d), dtype=q.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_attention_decode(stream, q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), out.data_ptr(), m, hq,
                                          cache.kv_heads, d, offset, _lib.ptr(offset_dev), max_len, 1.0 / math.sqrt(d),
                                          ws.data_ptr(), ws.numel(), _lib.dtype_code(q.dtype))
    _lib.check(rc, "mt_attention_decode")
    return out


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, offset: int = 0,
              offsets: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(q k^T / sqrt(d) + causal mask) v for batches of sequences and prefill-sized inputs
    (examples/llama3_70b.py:103-115): q [B, M, hq, d] (rotated), k_cache / v_cache [B, capacity, hkv, d] with the M new
    tokens of every sequence already appended at rows offset_b .. offset_b + M - 1; returns [B, M, hq * d].  ``offsets``
    (int32 [B] on the device) gives every sequence its own number of cached positions, else ``offset`` holds for all.
    Any head size that is a multiple of 32 up to 256."""
    dev = _lib.require_cuda(q, k_cache, v_cache, offsets)
    if q.dim() != 4 or k_cache.dim() != 4 or k_cache.shape != v_cache.shape:
        raise ValueError("q must be [B, M, hq, d] and the caches [B, capacity, hkv, d]")
    b, m, hq, d = q.shape
    b2, capacity, hkv, d2 = k_cache.shape
    if b2 != b or d2 != d or hq % hkv != 0 or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise ValueError("q and the caches disagree on batch, head size, head grouping or dtype")
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("q and the caches must be contiguous")
    if offsets is not None and (offsets.dtype != torch.int32 or tuple(offsets.shape) != (b,)):
        raise ValueError("offsets must be int32 [B]")
    if out is None:
        out = torch.empty((b, m, hq * d), dtype=q.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib.mt_attention(_lib.current_stream(dev), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                   _lib.ptr(offsets), b, m, hq, hkv, d, offset, capacity, 1.0 / math.sqrt(d), _lib.dtype_code(q.dtype))
    _lib.check(rc, "mt_attention")
    return out


def fuse_columns(linears) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor, Optional[torch.Tensor]]:
    """Load-time: GPTQ linears with the same K, groups and bits side by side as one linear (q | k | v)."""
    qw = torch.cat([l.qweight for l in linears], dim=1).contiguous()
    qz = torch.cat([l.qzeros for l in linears], dim=1).contiguous()
    sc = torch.cat([l.scales for l in linears], dim=1).contiguous()
    biases = [getattr(l, "bias", None) for l in linears]
    bi = torch.cat(biases).contiguous() if all(isinstance(b, torch.Tensor) for b in biases) else None
    return qw, qz, sc, bi


class RMSNorm(Module):
    def __init__(self, size: int, eps: float = 1e-5, dtype: str = "float16") -> None:
        super().__init__()
        self.eps = eps
        self.weight = self.register_buffer("weight", (size,), dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight, self.eps)


class QAttention(Module):
    """``Attention(hidden_size, nr_querys, nr_groups, head_size)`` of the reference on GPTQ linears
    (``nr_groups`` = query heads per kv head, as there).  ``forward`` takes the M new tokens of one sequence
    [M, hidden], the layer's cache and the position of the first token."""

    def __init__(self, hidden_size: int, nr_querys: int, nr_groups: int, head_size: int, quant_groups: int, bits: int = 8,
                 bias: bool = False, dtype: str = "float16") -> None:
        super().__init__()
        cls = QLinearWithBias if bias else QLinear
        self.nr_querys, self.nr_kv, self.head_size, self.bits = nr_querys, nr_querys // nr_groups, head_size, bits
        self.q_proj = self.register_module("q_proj", cls(hidden_size, nr_querys * head_size, quant_groups, bits, dtype))
        self.k_proj = self.register_module("k_proj", cls(hidden_size, self.nr_kv * head_size, quant_groups, bits, dtype))
        self.v_proj = self.register_module("v_proj", cls(hidden_size, self.nr_kv * head_size, quant_groups, bits, dtype))
        self.o_proj = self.register_module("o_proj", QLinear(nr_querys * head_size, hidden_size,
                                                             quant_groups * (nr_querys * head_size) // hidden_size, bits, dtype))
        self._qkv = None

    def update_buffer(self, name: str, value, sharded: bool = False) -> None:
        super().update_buffer(name, value, sharded)
        self._qkv = None

    def forward(self, x: torch.Tensor, cache: KVCache, cos: torch.Tensor, sin: torch.Tensor, offset: int,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._qkv is None:
            for lin in (self.q_proj, self.k_proj, self.v_proj):
                if lin._groups() is not None:
                    raise ValueError("act-order q / k / v projections are not fused")
            self._qkv = fuse_columns((self.q_proj, self.k_proj, self.v_proj))
        qw, qz, sc, bi = self._qkv
        q = qkv_rope_append(x, qw, qz, sc, cos, sin, cache, self.nr_querys, offset, bits=self.bits, bias=bi)
        m = x.shape[0]
        if self.head_size == 128 and self.nr_querys // self.nr_kv <= 8 and m <= 16:
            a = attention_decode(q, cache, offset)                 # split over the cached positions: the decode kernel
        else:                                                      # prefill-sized inputs and other head sizes: one warp per query row
            a = attention(q.unsqueeze(0), cache.k.unsqueeze(0), cache.v.unsqueeze(0), offset).view(m, -1)
        cache.length = max(cache.length, offset + m)
        o = self.o_proj
        if residual is None:
            return o._matmul(a, None)
        return quantized_matrix_multiply_residual(a, o.qweight, o.qzeros, o.scales, o._groups(), residual, bits=self.bits)


class QDecoderLayer(Module):
    """``TransformerBlock`` of the reference (examples/llama3_70b.py:144-162) with the same child names."""

    def __init__(self, hidden_size: int, nr_querys: int, nr_groups: int, head_size: int, internal_size: int, bits: int = 4,
                 group_size: int = 128, eps: float = 1e-5, dtype: str = "float16") -> None:
        super().__init__()
        self.self_attn = self.register_module("self_attn", QAttention(hidden_size, nr_querys, nr_groups, head_size,
                                                                      hidden_size // group_size, bits, False, dtype))
        self.mlp = self.register_module("mlp", QFeedForward(hidden_size, internal_size, hidden_size // group_size,
                                                            internal_size // group_size, bits, False, dtype=dtype))
        self.input_layernorm = self.register_module("input_layernorm", RMSNorm(hidden_size, eps, dtype))
        self.post_attention_layernorm = self.register_module("post_attention_layernorm", RMSNorm(hidden_size, eps, dtype))

    def forward(self, x: torch.Tensor, cache: KVCache, cos: torch.Tensor, sin: torch.Tensor, offset: int) -> torch.Tensor:
        h = self.self_attn(self.input_layernorm(x), cache, cos, sin, offset, residual=x)      # x + attention_output
        return self.mlp(self.post_attention_layernorm(h), residual=h)                           # + ffn_output
