"""sigmoid, RMS norm, rotary embedding and softmax (minit/functional/special.py:6-26).  The formulas follow the
reference's kernels: fp32 arithmetic inside, one rounding to the tensor's dtype at the end
(minit/cuda/kernel/cuda/rms_norm.py:55-99, rope.py:58-84, softmax.py:55-114)."""
from __future__ import annotations

import torch

from .utils import unwrap, wrap

__all__ = ["sigmoid", "rms_norm", "rope", "softmax"]


def sigmoid(x):
    t = unwrap(x)
    return wrap((1.0 / (1.0 + torch.exp(-t.float()))).to(t.dtype))


def rms_norm(x, weight, axis: int, eps: float):
    assert isinstance(eps, float) and 0 < eps < 0.5
    t, w = unwrap(x), unwrap(weight)
    assert w.dim() == 1 and w.shape[0] == t.shape[axis]
    f = t.float()
    scale = torch.rsqrt(f.pow(2).mean(dim=axis, keepdim=True) + eps)
    shape = [1] * t.dim()
    shape[axis] = w.shape[0]
    return wrap((f * scale * w.float().view(shape)).to(t.dtype))


def rope(x, freqs_cos, freqs_sin):
    """x [batch, seq, heads, head_size]: element pairs (2i, 2i + 1) are rotated by the angle of (position, i);
    the tables are [seq, head_size / 2]."""
    t = unwrap(x)
    b, s, h, d = t.shape
    cos = unwrap(freqs_cos).float().view(1, s, 1, d // 2)
    sin = unwrap(freqs_sin).float().view(1, s, 1, d // 2)
    pairs = t.float().view(b, s, h, d // 2, 2)
    re, im = pairs[..., 0], pairs[..., 1]
    out = torch.stack((re * cos - im * sin, im * cos + re * sin), dim=-1)
    return wrap(out.view(b, s, h, d).to(t.dtype))


def softmax(x, axis: int):
    t = unwrap(x)
    return wrap(torch.softmax(t.float(), dim=axis).to(t.dtype))
