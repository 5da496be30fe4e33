"""CPU restatement of MiniT's quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA path is compared against.  Nothing in
the shipped package imports it: only the test-suite, the smoke check and the
CPU-baseline legs of the benchmark may call it.

Parity status: the reference ships no tests, golden vectors or fixtures for this
path, so parity is *unpinned by reference tests*.  It is pinned instead against
outputs of the reference's own ``dispatch_dequantize`` executed on CPU; those
outputs are committed as fixtures (``tests/golden/*.npz``, produced by
``tests/golden/make_golden.py``).

The steps that restate CUDA kernel strings of the reference (``unpack_*`` + ``qlinear`` as the fused kernel of
``examples/qwen1_5_int8.py:156-216``, ``rms_norm``, ``rope``, the softmax inside ``attention``) are pinned against
outputs of those strings, compiled unchanged for sm_100a (``oracle/build_ref_cuda.py``) and run on a B200:
``tests/golden/ref_cuda_golden.npz``, made by ``tests/golden/make_cuda_golden.py``, checked in ``tests/test_oracle.py``.
``unpack_rows`` / ``unpack_cols`` are also pinned against the reference's own Python ``unpack`` run on CPU (same
fixture script as the dequantizer).  Still *unpinned*: ``sigmoid`` / ``silu`` / ``swiglu`` / ``add_residual`` (an
expression of the reference's generic elementwise generator, not a kernel string of its own); they are checked by
construction properties (``tests/test_oracle.py``).

What each function follows in the reference (paths relative to the reference
project root):

* ``unpack_rows`` / ``unpack_cols`` -- ``examples/qwen1_5_int8.py:40-50``
  (``unpack``: little-endian elements inside each int32) and the bit-width
  generic accessors ``ColPackedMatrix`` / ``RowPackedMatrix`` at
  ``examples/qwen1_5_int8.py:97-138`` (``(word >> (i % pack) * bits) & mask``).
* ``dequantize`` -- ``minit/quantize/dispatch.py:14-20``:
  ``(data.cast(T) - (zero.cast(T) + 1)) * scale`` with ``scale``/``zero``
  gathered along K by ``group`` (``minit/quantize/tensor.py:29-30`` fixes the
  axis to 0) and ``T`` the dtype of ``scale``.
* ``qlinear`` -- orientation ``out[M,N] = x[M,K] @ W[K,N]`` from the fused kernel
  ``examples/qwen1_5_int8.py:156-200``; fp32 accumulation from
  ``minit/cuda/kernel/cublas.py:122-127`` (``CUBLAS_COMPUTE_32F``); the bias add
  of ``QLinearWithBias.forward`` ``examples/qwen1_5_int8.py:311-317``.
* ``sigmoid`` / ``silu`` / ``swiglu`` / ``add_residual`` -- the elementwise rules of
  ``minit/cuda/dispatch.py:135-143`` (``{0} + {1}``, ``{0} * {1}`` in the tensor dtype;
  sigmoid ``1.0 / (1.0 + expf((float)-{0}))`` cast to the tensor dtype), composed as
  ``silu(x) = x * sigmoid(x)`` (``examples/llama3_70b.py:44-45``) and
  ``down(silu(gate(x)) * up(x))`` (``examples/llama3_70b.py:126-130``); the residual add is
  ``x + attention_output`` (``examples/llama3_70b.py:160-162``).  Every step rounds to the tensor dtype.
* ``interleave_gate_up`` -- no counterpart in the reference: the column order this build's fused
  gate / up linear uses (blocks of eight = four gate, four up columns), restated in numpy.
* ``rms_norm`` -- ``minit/cuda/kernel/cuda/rms_norm.py:55-91``: fp32 sum of squares, ``sqrt(mean + eps)``,
  ``value / rms * weight`` in fp32, one rounding.
* ``rope`` -- ``minit/cuda/kernel/cuda/rope.py:58-73``: pairs ``(x[2i], x[2i+1])`` rotated by fp32
  ``(cos, sin)[position, i]``; tables as built at ``examples/llama3_70b.py:206-212`` (rounded to the tensor dtype).
* ``attention`` -- ``examples/llama3_70b.py:85-115`` step by step, each step rounded to the tensor dtype:
  scores (fp32 accumulate), ``/ sqrt(d)``, ``+ mask``, softmax (``minit/cuda/kernel/cuda/softmax.py:55-106``:
  fp32 max, exp, sum, divide), weighted sum of v; query head n reads kv head ``n // nr_groups``.
* ``shard_*`` -- the tensor-parallel rules ``minit/collective/dispatch.py:26-37``
  and the local slice of ``minit/collective/tensor.py:88-94``.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = [
    "pack_rows", "pack_cols", "unpack_rows", "unpack_cols", "dequantize",
    "dequantize_packed", "qlinear", "w8_perchannel_as_gptq", "w8_perchannel_linear",
    "shard_column", "shard_row", "make_gptq_case", "make_w8_case", "tolerance_ok",
    "sigmoid", "silu", "swiglu", "add_residual", "interleave_columns", "interleave_gate_up",
    "rms_norm", "rope_tables", "rope", "attention",
]


def _pack_size(bits: int) -> int:
    assert bits in (4, 8)
    return 32 // bits


# ---------------------------------------------------------------------------
# packing (integer, bit exact)
# ---------------------------------------------------------------------------
def pack_rows(q: np.ndarray, bits: int) -> np.ndarray:
    """[K,N] uint8 -> int32 [K/pack,N]; element k sits at bits ((k % pack)*bits) of word k//pack."""
    ps = _pack_size(bits)
    k, n = q.shape
    assert k % ps == 0
    q = q.astype(np.uint32).reshape(k // ps, ps, n)
    word = np.zeros((k // ps, n), dtype=np.uint32)
    for j in range(ps):
        word |= q[:, j, :] << np.uint32(j * bits)
    return word.view(np.int32)


def pack_cols(z: np.ndarray, bits: int) -> np.ndarray:
    """[G,N] uint8 -> int32 [G,N/pack]; element n sits at bits ((n % pack)*bits) of word n//pack."""
    ps = _pack_size(bits)
    g, n = z.shape
    assert n % ps == 0
    z = z.astype(np.uint32).reshape(g, n // ps, ps)
    word = np.zeros((g, n // ps), dtype=np.uint32)
    for j in range(ps):
        word |= z[:, :, j] << np.uint32(j * bits)
    return word.view(np.int32)


def unpack_rows(qweight: np.ndarray, bits: int) -> np.ndarray:
    """int32 [K/pack,N] -> uint8 [K,N] (ColPackedMatrix, examples/qwen1_5_int8.py:119-138)."""
    ps = _pack_size(bits)
    w = np.ascontiguousarray(qweight).view(np.uint32)
    kp, n = w.shape
    mask = np.uint32((1 << bits) - 1)
    out = np.empty((kp, ps, n), dtype=np.uint8)
    for j in range(ps):
        out[:, j, :] = ((w >> np.uint32(j * bits)) & mask).astype(np.uint8)
    return out.reshape(kp * ps, n)


def unpack_cols(qzeros: np.ndarray, bits: int) -> np.ndarray:
    """int32 [G,N/pack] -> uint8 [G,N] (RowPackedMatrix, examples/qwen1_5_int8.py:97-116)."""
    ps = _pack_size(bits)
    w = np.ascontiguousarray(qzeros).view(np.uint32)
    g, npk = w.shape
    mask = np.uint32((1 << bits) - 1)
    out = np.empty((g, npk, ps), dtype=np.uint8)
    for j in range(ps):
        out[:, :, j] = ((w >> np.uint32(j * bits)) & mask).astype(np.uint8)
    return out.reshape(g, npk * ps)


# ---------------------------------------------------------------------------
# dequantisation (bit exact in the scale dtype)
# ---------------------------------------------------------------------------
def dequantize(q: np.ndarray, g_idx: np.ndarray, z: np.ndarray, scales: torch.Tensor) -> torch.Tensor:
    """W[k,n] = (T(q[k,n]) - (T(z[g[k],n]) + 1)) * s[g[k],n], every step in T = scales.dtype.

    Follows minit/quantize/dispatch.py:14-20 operation by operation (gather, cast,
    add 1, subtract, multiply), each one rounding to T like the reference's
    elementwise kernels do.
    """
    assert scales.dtype in (torch.float16, torch.bfloat16)
    t = scales.dtype
    gi = torch.from_numpy(np.ascontiguousarray(g_idx).astype(np.int64))
    s = scales.index_select(0, gi)
    zz = torch.from_numpy(np.ascontiguousarray(z)).index_select(0, gi)
    data = torch.from_numpy(np.ascontiguousarray(q)).to(t)
    zero = zz.to(t) + torch.ones((), dtype=t)
    return (data - zero) * s


def dequantize_packed(qweight, g_idx, qzeros, scales: torch.Tensor, bits: int) -> torch.Tensor:
    """Packed GPTQ tensors -> W[K,N].  g_idx None means k // (K/G); qzeros None means
    the symmetric midpoint (stored zero 2**(bits-1) - 1, so zero+1 is the midpoint)."""
    qweight = _np(qweight)
    q = unpack_rows(qweight, bits)
    k, n = q.shape
    g = scales.shape[0]
    if g_idx is None:
        assert k % g == 0
        g_idx = np.arange(k, dtype=np.int32) // (k // g)
    else:
        g_idx = _np(g_idx)
    if qzeros is None:
        z = np.full((g, n), (1 << (bits - 1)) - 1, dtype=np.uint8)
    else:
        z = unpack_cols(_np(qzeros), bits)
    return dequantize(q, g_idx, z, scales)


def _np(a):
    if isinstance(a, torch.Tensor):
        return a.detach().cpu().numpy()
    return np.asarray(a)


# ---------------------------------------------------------------------------
# linear
# ---------------------------------------------------------------------------
def qlinear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """out = T( float(x) @ float(W) [+ float(bias)] ): dequantize-then-matmul with fp32 accumulate."""
    acc = x.float() @ w.float()
    if bias is not None:
        acc = acc + bias.float()
    return acc.to(x.dtype)


def w8_perchannel_as_gptq(w_i8: np.ndarray, scales: torch.Tensor):
    """int8 per-output-channel weights expressed in the reference's GPTQ-8bit layout:
    q = w + 128 packed four per word along K, one group, stored zero 127 (so zero+1 = 128)."""
    k, n = w_i8.shape
    q = (w_i8.astype(np.int16) + 128).astype(np.uint8)
    qweight = pack_rows(q, 8)
    qzeros = pack_cols(np.full((1, n), 127, dtype=np.uint8), 8)
    g_idx = np.zeros((k,), dtype=np.int32)
    return qweight, g_idx, qzeros, scales.reshape(1, n)


def w8_perchannel_linear(x: torch.Tensor, w_i8: np.ndarray, scales: torch.Tensor, bias=None) -> torch.Tensor:
    qweight, g_idx, qzeros, s = w8_perchannel_as_gptq(w_i8, scales)
    return qlinear(x, dequantize_packed(qweight, g_idx, qzeros, s, 8), bias)


# ---------------------------------------------------------------------------
# the elementwise steps around the linears of a gated feed-forward
# ---------------------------------------------------------------------------
def sigmoid(x: torch.Tensor) -> torch.Tensor:
    """T(1.0 / (1.0 + expf(float(-x)))): fp32 exp, the division in double (the literals are doubles)."""
    e = torch.exp((-x).float()).double()
    return (1.0 / (1.0 + e)).to(x.dtype)


def silu(x: torch.Tensor) -> torch.Tensor:
    return (x.float() * sigmoid(x).float()).to(x.dtype)          # one multiply in T: exact product, one rounding


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """T(silu(gate) * up), silu itself already rounded to T (three roundings after the linears)."""
    return (silu(gate).float() * up.float()).to(gate.dtype)


def add_residual(residual: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return (residual.float() + y.float()).to(y.dtype)


def interleave_columns(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """[R, H], [R, H] -> [R, 2H]: output column c = a[:, 4 (c // 8) + c % 8] if c % 8 < 4 else b[:, 4 (c // 8) + c % 8 - 4]."""
    r, h = a.shape
    out = np.empty((r, 2 * h), dtype=a.dtype)
    o = out.reshape(r, h // 4, 8)
    o[:, :, :4] = a.reshape(r, h // 4, 4)
    o[:, :, 4:] = b.reshape(r, h // 4, 4)
    return out


def interleave_gate_up(gate, up, bits: int):
    """(qweight, qzeros, scales) of the gate and up linears -> the same three for the fused linear."""
    gq, gz, gs = (_np(t) for t in gate)
    uq, uz, us = (_np(t) for t in up)
    qw = interleave_columns(gq, uq)
    sc = interleave_columns(gs.view(np.uint16) if gs.dtype != np.uint16 else gs, us.view(np.uint16) if us.dtype != np.uint16 else us)
    z = interleave_columns(unpack_cols(gz, bits), unpack_cols(uz, bits))
    return qw, pack_cols(z, bits), sc


# ---------------------------------------------------------------------------
# the steps either side of the linears in a decoder layer
# ---------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    rms = torch.sqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf / rms * weight.float()).to(x.dtype)


def rope_tables(head_size: int, size: int, theta: float = 5e5, dtype=torch.float16):
    freqs = (1.0 / theta) ** (torch.arange(0, head_size // 2, dtype=torch.float32) * (2.0 / head_size))
    ang = torch.arange(0, size, dtype=torch.float32)[:, None] * freqs[None, :]
    return ang.cos().to(dtype).float(), ang.sin().to(dtype).float()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int) -> torch.Tensor:
    """x [S, heads, D]; token s is at position offset + s."""
    s_len, _, d = x.shape
    xf = x.float().reshape(s_len, -1, d // 2, 2)
    re, im = xf[..., 0], xf[..., 1]
    c = cos[offset:offset + s_len][:, None, :]
    sn = sin[offset:offset + s_len][:, None, :]
    out = torch.stack((re * c - im * sn, im * c + re * sn), dim=-1)
    return out.reshape(x.shape).to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, offset: int) -> torch.Tensor:
    """q [S, hq, D] (rotated), k / v [offset + S, hkv, D] (the cache including the new tokens) -> [S, hq * D]."""
    T = q.dtype
    s_len, hq, d = q.shape
    hkv = k.shape[1]
    r = hq // hkv
    kk = k.repeat_interleave(r, dim=1).float()                       # "bs(hd)->bs(hr)d"
    vv = v.repeat_interleave(r, dim=1).float()
    qk = torch.einsum("snd,tnd->nst", q.float(), kk).to(T)
    qk = (qk.float() / float(np.sqrt(d))).to(T)
    t_len = k.shape[0]
    mask = torch.zeros((s_len, t_len))
    for i in range(s_len):
        mask[i, offset + i + 1:] = -np.inf
    qk = (qk.float() + mask[None]).to(T)
    p = torch.softmax(qk.float(), dim=-1).to(T)
    out = torch.einsum("nst,tnd->snd", p.float(), vv).to(T)
    return out.reshape(s_len, hq * d)


# ---------------------------------------------------------------------------
# tensor-parallel sharding of GPTQ tensors
# ---------------------------------------------------------------------------
def shard_column(qweight, qzeros, scales, bits: int, rank: int, size: int):
    """Weight split on out-features (minit/collective/dispatch.py:26-30): slice N."""
    ps = _pack_size(bits)
    n = qweight.shape[1]
    assert n % (size * ps) == 0
    lo, hi = n // size * rank, n // size * (rank + 1)
    return qweight[:, lo:hi], qzeros[:, lo // ps:hi // ps], scales[:, lo:hi]


def shard_row(qweight, qzeros, scales, bits: int, rank: int, size: int):
    """Weight split on in-features (minit/collective/dispatch.py:33-37): slice K on group
    boundaries (no act-order); the caller slices x on K the same way and sums partials."""
    ps = _pack_size(bits)
    kp = qweight.shape[0]
    g = scales.shape[0]
    assert kp % size == 0 and g % size == 0
    return (qweight[kp // size * rank:kp // size * (rank + 1)],
            qzeros[g // size * rank:g // size * (rank + 1)],
            scales[g // size * rank:g // size * (rank + 1)])


# ---------------------------------------------------------------------------
# seeded synthetic cases (generated on CPU so every consumer sees the same bits)
# ---------------------------------------------------------------------------
def make_gptq_case(k: int, n: int, m: int, bits: int = 4, group_size: int = 128,
                   act_order: bool = False, dtype=torch.float16, seed: int = 0,
                   scale_lo: float = 0.002, scale_hi: float = 0.02, bias: bool = False):
    gen = torch.Generator().manual_seed(seed)
    g = k // group_size
    q = torch.randint(0, 1 << bits, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    z = torch.randint(0, 1 << bits, (g, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    scales = (scale_lo + (scale_hi - scale_lo) * torch.rand((g, n), generator=gen)).to(dtype)
    g_idx = (torch.arange(k) // group_size).to(torch.int32)
    if act_order:
        g_idx = g_idx[torch.randperm(k, generator=gen)]
    x = torch.randn((m, k), generator=gen).to(dtype)
    case = dict(
        qweight=torch.from_numpy(pack_rows(q, bits)), qzeros=torch.from_numpy(pack_cols(z, bits)),
        scales=scales, g_idx=g_idx.contiguous(), x=x, bits=bits, q=q, z=z,
    )
    if bias:
        case["bias"] = torch.randn((n,), generator=gen).to(dtype)
    return case


def make_w8_case(k: int, n: int, m: int, dtype=torch.float16, seed: int = 0):
    gen = torch.Generator().manual_seed(seed)
    w = torch.randint(-127, 128, (k, n), generator=gen, dtype=torch.int32).to(torch.int8)
    scales = (0.001 + 0.009 * torch.rand((n,), generator=gen)).to(dtype)
    x = torch.randn((m, k), generator=gen).to(dtype)
    return dict(w=w, scales=scales, x=x)


def tolerance_ok(out: torch.Tensor, ref: torch.Tensor, factor: float = 1e-2):
    """max|out - ref| <= factor * rms(ref); returns (ok, max_abs_err, bound)."""
    o, r = out.float().cpu(), ref.float().cpu()
    err = (o - r).abs().max().item() if r.numel() else 0.0
    bound = factor * r.pow(2).mean().sqrt().item() if r.numel() else 0.0
    return err <= bound, err, bound
