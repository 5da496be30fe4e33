"""Helpers shared by the GPU parity tests: move oracle cases to the device, run the oracle."""
import numpy as np
import torch

from oracle import qlinear_oracle as O


def to_dev(case, dev="cuda:0"):
    out = {}
    for k, v in case.items():
        out[k] = v.to(dev) if isinstance(v, torch.Tensor) else v
    return out


def oracle_w(case, act_order):
    return O.dequantize_packed(case["qweight"], case["g_idx"] if act_order else None, case["qzeros"], case["scales"], case["bits"])


def oracle_out(case, act_order, bias=None):
    return O.qlinear(case["x"], oracle_w(case, act_order), bias)


def assert_close(out, ref, what=""):
    """fp16: the north-star bound, max|out - ref| <= 1e-2 * rms(ref).
    bf16: the same bound plus one bf16 ulp of the largest reference value (at most 2^-7 * max|ref|):
    a bf16 result is rounded to 8 significant bits, so two correct fp32 sums that differ in
    the last place round to neighbouring bf16 values, and one such step at |v| ~ 4 (0.031) is
    already larger than 1e-2 * rms for these shapes."""
    ok, err, bound = O.tolerance_ok(out, ref, 1e-2)
    if ref.dtype == torch.bfloat16 and ref.numel():
        bound = bound + ref.float().abs().max().item() * 2.0 ** -7
        ok = err <= bound
    assert ok, f"{what}: max abs err {err:.4g} > bound {bound:.4g}"
    return err, bound
