"""Run the reference's own CUDA kernels (the libraries oracle/build_ref_cuda.py builds from the reference's source
strings) on a GPU and store their outputs as a fixture, so that the CPU oracle can be checked against what the
reference computes rather than against a reading of it.

    python tests/golden/make_cuda_golden.py <output directory>

writes ``ref_cuda_golden.npz`` (inputs and outputs of every case) and ``ref_cuda_timing.json`` (the reference's fused
kernel, 8-bit 4096 x 4096, at 1 and 16 rows: the "kernel to beat").  Shapes are the ones the reference's host code
accepts (N and K multiples of its 32-wide tile, group indices in range): its device code asserts on anything else.
Inputs come from the oracle's seeded generators.  The kernels: the fused 8-bit GPTQ linear `qmm_*`
(examples/qwen1_5_int8.py:156-216; output zeroed first as its wrapper does, :262-263), `rms_norm`
(minit/cuda/kernel/cuda/rms_norm.py:56-97), `rope` (.../rope.py:57-85, instantiated for float) and `softmax`
(.../softmax.py:55-114).
"""
import ctypes
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import qlinear_oracle as O  # noqa: E402

REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "oracle", "_ref")
vp, ci, cs, cd = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_double


def load(lib, name, argtypes):
    fn = getattr(ctypes.CDLL(os.path.join(REF, lib)), name)
    fn.restype, fn.argtypes = None, argtypes
    return fn


def main(out_dir):
    dev = torch.device("cuda", 0)
    os.makedirs(out_dir, exist_ok=True)
    qmm = load("libref_qmm_f16.so", "qmm_ref", [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci])
    rms = load("libref_rms_norm_f16.so", "minit_rms_norm", [vp, vp, vp, vp, cs, cs, cs, cd])
    rope = load("libref_rope_f32.so", "minit_rope", [vp, vp, vp, vp, vp, cs, cs, cs, cs])
    smx = load("libref_softmax_f16.so", "minit_softmax", [vp, vp, vp, cs, cs, cs])
    fix = {}

    def run_qmm(c, m, n, k):
        d = {key: (v.to(dev) if isinstance(v, torch.Tensor) else v) for key, v in c.items()}
        out = torch.zeros((m, n), dtype=torch.float16, device=dev)           # the wrapper zeroes the output: the kernel adds into it
        qmm(None, d["x"].data_ptr(), d["qweight"].data_ptr(), d["g_idx"].data_ptr(), d["qzeros"].data_ptr(), d["scales"].data_ptr(),
            out.data_ptr(), m, n, k, d["scales"].shape[0])
        torch.cuda.synchronize()
        return d, out

    # ---- fused 8-bit linear: contiguous groups, act-order, several rows ----
    for i, (k, n, m, gs, act) in enumerate([(256, 128, 1, 128, False), (512, 256, 3, 64, True), (1024, 512, 16, 128, False), (2048, 96, 2, 128, True)]):
        c = O.make_gptq_case(k, n, m, bits=8, group_size=gs, act_order=act, seed=900 + i)
        _, out = run_qmm(c, m, n, k)
        for key in ("x", "scales"):
            fix[f"qmm{i}_{key}"] = c[key].view(torch.int16).numpy()
        for key in ("qweight", "qzeros", "g_idx"):
            fix[f"qmm{i}_{key}"] = c[key].numpy()
        fix[f"qmm{i}_out"] = out.cpu().view(torch.int16).numpy()

    # ---- rms_norm over the middle axis of [a, b, c] ----
    gen = torch.Generator().manual_seed(77)
    for i, (a, b, c3) in enumerate([(4, 1024, 1), (2, 96, 3), (1, 8192, 1)]):
        x = (torch.randn((a, b, c3), generator=gen) * 1.5).half()
        w = (1.0 + 0.1 * torch.randn((b,), generator=gen)).half()
        xd, wd = x.to(dev), w.to(dev)
        y = torch.empty_like(xd)
        rms(None, xd.data_ptr(), wd.data_ptr(), y.data_ptr(), a, b, c3, 1e-5)
        torch.cuda.synchronize()
        fix[f"rms{i}_x"], fix[f"rms{i}_w"], fix[f"rms{i}_out"] = x.view(torch.int16).numpy(), w.view(torch.int16).numpy(), y.cpu().view(torch.int16).numpy()

    # ---- rope on [batch, seqlen, heads, head_size] with [seqlen, head_size / 2] tables ----
    for i, (bs, sl, nh, hs) in enumerate([(1, 5, 4, 64), (2, 3, 2, 128)]):
        x = torch.randn((bs, sl, nh, hs), generator=gen)
        cos, sin = O.rope_tables(hs, sl, dtype=torch.float32)
        xd, cd_, sd = x.to(dev), cos.contiguous().to(dev), sin.contiguous().to(dev)
        y = torch.empty_like(xd)
        rope(None, xd.data_ptr(), cd_.data_ptr(), sd.data_ptr(), y.data_ptr(), bs, sl, nh, hs)
        torch.cuda.synchronize()
        fix[f"rope{i}_x"], fix[f"rope{i}_cos"], fix[f"rope{i}_sin"], fix[f"rope{i}_out"] = x.numpy(), cos.numpy(), sin.numpy(), y.cpu().numpy()

    # ---- softmax over the middle axis of [a, b, c] ----
    for i, (a, b, c3) in enumerate([(3, 100, 1), (2, 40, 4), (1, 4097, 1)]):
        x = (torch.randn((a, b, c3), generator=gen) * 3.0).half()
        if i == 0:
            x[0, 50:, 0] = float("-inf")                                     # a causal-mask row: masked positions are -inf
        xd = x.to(dev)
        y = torch.empty_like(xd)
        smx(None, xd.data_ptr(), y.data_ptr(), a, b, c3)
        torch.cuda.synchronize()
        fix[f"smx{i}_x"], fix[f"smx{i}_out"] = x.view(torch.int16).numpy(), y.cpu().view(torch.int16).numpy()

    np.savez_compressed(os.path.join(out_dir, "ref_cuda_golden.npz"), **fix)

    # ---- the kernel to beat: 8-bit 4096 x 4096, one and sixteen rows, zeroing included as in the wrapper ----
    timing = {"gpu": torch.cuda.get_device_name(0), "shape": [4096, 4096], "bits": 8, "group_size": 128}
    for m in (1, 16):
        c = O.make_gptq_case(4096, 4096, m, bits=8, seed=950 + m)
        d = {key: (v.to(dev) if isinstance(v, torch.Tensor) else v) for key, v in c.items()}
        out = torch.zeros((m, 4096), dtype=torch.float16, device=dev)

        def call():
            out.zero_()
            qmm(None, d["x"].data_ptr(), d["qweight"].data_ptr(), d["g_idx"].data_ptr(), d["qzeros"].data_ptr(), d["scales"].data_ptr(),
                out.data_ptr(), m, 4096, 4096, 32)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            call()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 20
        ref = O.qlinear(c["x"], O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 8))
        ok, err, bound = O.tolerance_ok(out.cpu(), ref, 1e-2)
        timing[f"m{m}"] = {"us_per_call": us, "weight_GBps": (4096 * 4096 + 2 * 32 * 4096 + 32 * 4096) / us / 1e3,
                           "max_err_vs_oracle": err, "bound_1e-2_rms": bound}
    with open(os.path.join(out_dir, "ref_cuda_timing.json"), "w") as f:
        json.dump(timing, f, indent=1)
    print(json.dumps(timing))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else ".")
