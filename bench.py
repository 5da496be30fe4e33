#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch M]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload): the GPTQ int4 (group 128) linears of Llama-3-70B at decode batch
M (default 1), tensor-parallel over N GPUs: per layer qkv (8192 -> 10240/N, column-parallel),
o (8192/N -> 8192, row-parallel + all-reduce), fused gate/up (8192 -> 57344/N, column-parallel),
down (28672/N -> 8192, row-parallel + all-reduce); 80 layers, distinct random weights per layer
(35.6 GB at N=1, far larger than L2).  One step = one pass over all 80 layers.  Strong
scaling: the total work is fixed, each rank holds 1/N of every weight.

Metric: aggregate weight GB/s = packed weight bytes (qweight + qzeros + scales) of all ranks
read per step / step time (device time, CUDA events, max over ranks).

The reference arm (--impl reference) times the reference's dequantize-then-matmul restated on
the host CPU (oracle/, torch with all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, Q_HEADS, KV_HEADS, HEAD_DIM, LAYERS, GROUP = 8192, 28672, 64, 8, 128, 80, 128
BITS = 4


def layer_shapes(tp: int):
    """(name, K, N, kind) of one rank's four linears."""
    qkv_n = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM
    return [("qkv", HIDDEN, qkv_n // tp, "column"), ("o", HIDDEN // tp, HIDDEN, "row"),
            ("gate_up", HIDDEN, 2 * INTER // tp, "column"), ("down", INTER // tp, HIDDEN, "row")]


def weight_bytes(k: int, n: int, bits: int = BITS, gs: int = GROUP) -> int:  # packed weights + scales + zeros
    g = k // gs
    return k * n * bits // 8 + g * n * 2 + g * n * bits // 8


def algorithmic_bytes(m: int, k: int, n: int) -> int:
    return weight_bytes(k, n) + 2 * m * k + 2 * m * n


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.path = f"/tmp/minit_b200_clocks_{os.getpid()}.csv"
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(index)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    sm.append(float(parts[0])); mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            busy = [s for s in sm if s > 0.5 * max(sm)]
            out["sm_mhz"] = statistics.median(busy or sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def run_mlp_block(args):
    """The feed-forward block of a decode step, down(silu(gate(x)) * up(x)) + residual on the Llama-3-70B shapes,
    timed with its elementwise steps as separate launches (gate/up linear, activation, down linear, residual add)
    and fused into the two linears.  Distinct weights per layer (more than L2), one CUDA graph per form."""
    import minit_b200 as M
    from minit_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    m, nl = args.m, min(args.layers, 8)
    gen = torch.Generator(device=dev).manual_seed(0)

    def rnd_linear(k, n):
        qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        sc = (0.002 + 0.018 * torch.rand((k // GROUP, n), device=dev, generator=gen)).half()
        return qw, qz, sc
    layers = [(rnd_linear(HIDDEN, 2 * INTER), rnd_linear(INTER, HIDDEN)) for _ in range(nl)]
    x = torch.randn((m, HIDDEN), device=dev).half()
    res = torch.randn((m, HIDDEN), device=dev).half()
    y = torch.empty((m, 2 * INTER), device=dev, dtype=torch.float16)
    h = torch.empty((m, INTER), device=dev, dtype=torch.float16)
    o = torch.empty((m, HIDDEN), device=dev, dtype=torch.float16)
    flags = _lib.FLAG_PDL if args.pdl else 0

    def separate():
        for (gq, gz, gs), (dq, dz, ds) in layers:
            M.quantized_matrix_multiply(x, gq, gz, gs, None, bits=BITS, out=y, flags=flags)
            hh = M.swiglu_interleaved(y)
            M.quantized_matrix_multiply(hh, dq, dz, ds, None, bits=BITS, out=o, flags=flags)
            torch.add(o, res, out=o)

    def fused():
        for (gq, gz, gs), (dq, dz, ds) in layers:
            M.quantized_gate_up_swiglu(x, gq, gz, gs, bits=BITS, out=h, flags=flags)
            M.quantized_matrix_multiply_residual(h, dq, dz, ds, None, res, bits=BITS, out=o, flags=flags)

    def timed(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(3, args.warmup)):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(args.steps):
                graph.replay()
            e1.record(side)
            torch.cuda.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        return e0.elapsed_time(e1) * 1e3 / (args.steps * nl)
    us_sep, us_fused = timed(separate), timed(fused)
    hbm_peak, kind = peaks()
    wb = weight_bytes(HIDDEN, 2 * INTER) + weight_bytes(INTER, HIDDEN)
    print(json.dumps({"mlp_block": "llama3-70b gate/up + silu*up + down + residual", "m": m, "layers": nl,
                      "us_per_block_separate": us_sep, "launches_separate": 4, "us_per_block_fused": us_fused, "launches_fused": 2,
                      "weight_GBps_fused": wb / us_fused / 1e3, "hbm_frac_fused": wb / us_fused / 1e3 / hbm_peak, "peak": kind,
                      "note": "weights of %d layers in rotation (%.1f GB), CUDA graph, PDL %s" % (nl, wb * nl / 1e9, "on" if args.pdl else "off")}))


def run_attention(args):
    """Decode attention alone (one token, Llama-3-70B heads) over `--context` cached positions: device time per call and
    the cache bytes it streams against the HBM peak.  Several caches in rotation, eager launches."""
    from minit_b200 import decoder as D
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ctx, m = args.context, args.m
    kvb = 2 * (ctx + m) * KV_HEADS * HEAD_DIM * 2
    copies = max(2, min(16, int(400e6 // kvb) + 1))
    caches = []
    for _ in range(copies):
        c = D.KVCache(ctx + m, KV_HEADS, HEAD_DIM, torch.float16, dev)
        c.k.normal_(); c.v.normal_()
        caches.append(c)
    q = torch.randn((m, Q_HEADS, HEAD_DIM), device=dev).half()
    out = torch.empty((m, Q_HEADS * HEAD_DIM), device=dev, dtype=torch.float16)

    def one():
        for c in caches:
            D.attention_decode(q, c, ctx, out=out)
    for _ in range(max(3, args.warmup)):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * copies)
    hbm_peak, kind = peaks()
    print(json.dumps({"attention_decode": "64 query / 8 kv heads x 128", "m": m, "context": ctx, "us_per_call": us,
                      "cache_GBps": kvb / us / 1e3, "hbm_frac": kvb / us / 1e3 / hbm_peak, "peak": kind,
                      "launch": "eager, %d caches in rotation (%.0f MB)" % (copies, kvb * copies / 1e6)}))


def run_decode_layer(args):
    """One token through whole decoder layers of Llama-3-70B (RMSNorm, fused qkv linear with rotary embedding + cache
    append, attention over `--context` cached positions, o_proj + residual, RMSNorm, fused feed-forward + residual): six
    launches per layer.  Distinct weights and caches per layer, one CUDA graph over all of them.  Under torchrun the
    layer is tensor parallel: heads and the feed-forward's inner dimension are split over the ranks, o_proj and
    down_proj run with the all-reduce and the residual add in the GEMV kernel."""
    import torch.distributed as dist
    import minit_b200 as M
    from minit_b200 import decoder as D
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(local_rank)
    far = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from minit_b200.collective import FusedAllReduce
        far = FusedAllReduce(m_max=max(16, args.m), n_max=HIDDEN)
    m, nl, ctx = args.m, min(args.layers, 16), args.context
    gen = torch.Generator(device=dev).manual_seed(rank)
    HQ, HKV = Q_HEADS // world, KV_HEADS // world
    inter = INTER // world

    def rnd_linear(k, n):
        qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        sc = (0.0005 + 0.001 * torch.rand((k // GROUP, n), device=dev, generator=gen)).half()
        return qw, qz, sc
    cos, sin = D.rope_tables(HEAD_DIM, ctx + m, 5e5, torch.float16, dev)
    layers = []
    for _ in range(nl):
        cache = D.KVCache(ctx + m, HKV, HEAD_DIM, torch.float16, dev)
        cache.k.normal_(generator=gen); cache.v.normal_(generator=gen)
        layers.append(dict(qkv=rnd_linear(HIDDEN, (HQ + 2 * HKV) * HEAD_DIM), o=rnd_linear(HQ * HEAD_DIM, HIDDEN),
                           gu=rnd_linear(HIDDEN, 2 * inter), dn=rnd_linear(inter, HIDDEN), cache=cache,
                           n1=torch.ones(HIDDEN, device=dev, dtype=torch.float16), n2=torch.ones(HIDDEN, device=dev, dtype=torch.float16)))
    x0 = torch.randn((m, HIDDEN), generator=torch.Generator().manual_seed(5)).half().to(dev)     # replicated
    flags = _flag_pdl() if args.pdl else 0

    def row_parallel(a, lin, residual):
        if far is not None:
            return far.matmul(a, *lin, None, bits=BITS, flags=flags, residual=residual)       # GEMV + all-reduce + residual, one kernel
        return M.quantized_matrix_multiply_residual(a, *lin, None, residual, bits=BITS, flags=flags)

    def step():
        x = x0
        for L in layers:
            xn = D.rms_norm(x, L["n1"])
            q = D.qkv_rope_append(xn, *L["qkv"], cos, sin, L["cache"], HQ, ctx, bits=BITS, flags=flags)
            a = D.attention_decode(q, L["cache"], ctx)
            h = row_parallel(a, L["o"], x)
            hn = D.rms_norm(h, L["n2"])
            g = M.quantized_gate_up_swiglu(hn, *L["gu"], bits=BITS, flags=flags)
            x = row_parallel(g, L["dn"], h)
        return x

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(args.steps):
            graph.replay()
        e1.record(side)
        barrier()
    torch.cuda.current_stream().wait_stream(side)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    us = ms.item() * 1e3 / (args.steps * nl)
    hbm_peak, kind = peaks()
    wb = sum(weight_bytes(k, n) for _, k, n, _ in layer_shapes(world))
    kvb = 2 * ctx * HKV * HEAD_DIM * 2
    if rank == 0:
        print(json.dumps({"decode_layer": "llama3-70b, int4 g128, tp%d" % world, "n_gpus": world, "m": m, "context": ctx, "layers_timed": nl,
                          "launches_per_layer": 6, "us_per_layer": us, "tokens_per_s_80_layers": m * 1e6 / (us * LAYERS),
                          "bytes_per_layer_per_gpu": wb + kvb, "hbm_frac": (wb + kvb) / us / 1e3 / hbm_peak, "peak": kind,
                          "note": "weights + KV cache of %d layers in rotation (%.1f GB per GPU), CUDA graph, max over ranks" % (nl, (wb + kvb) * nl / 1e9)}))
    if world > 1:
        from minit_b200 import _lib
        for ws in _lib._workspaces.values():
            assert _lib.workspace_error_word(ws) == 0, "a bounded wait of the fused all-reduce expired"
        dist.destroy_process_group()


def _flag_pdl():
    from minit_b200 import _lib
    return _lib.FLAG_PDL


def prefill_m4096(dev):
    """The other half of the headline metric: TFLOP/s of the int4 GEMM at M = 4096 on the prefill shapes
    (K, N) = (4096, 28672), (14336, 4096), (4096, 6144), against the measured dense bf16 tensor peak.
    Three weight sets in rotation, 3 warm-up and 10 timed launches per shape, CUDA events."""
    import minit_b200 as M
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak, kind = (float(json.load(open(path))["bf16_tflops"]), "measured cuBLAS bf16 burst") if os.path.exists(path) else (1590.0, "fallback")
    gen = torch.Generator(device=dev).manual_seed(99)
    mrows, shapes = 4096, []
    for k, n in [(4096, 28672), (14336, 4096), (4096, 6144)]:
        sets = []
        for _ in range(3):
            qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
            qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
            sc = (0.002 + 0.018 * torch.rand((k // GROUP, n), device=dev, generator=gen)).half()
            sets.append((qw, qz, sc))
        x = torch.randn((mrows, k), device=dev, generator=gen).half()
        out = torch.empty((mrows, n), device=dev, dtype=torch.float16)
        for i in range(3):
            M.quantized_matrix_multiply(x, *sets[i % 3], None, bits=BITS, out=out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(10):
            M.quantized_matrix_multiply(x, *sets[i % 3], None, bits=BITS, out=out)
        e1.record()
        torch.cuda.synchronize()
        tf = 2.0 * mrows * n * k * 10 / (e0.elapsed_time(e1) * 1e-3) / 1e12
        shapes.append({"k": k, "n": n, "tflops": tf, "frac": tf / peak})
        del sets, x, out
    return {"m": mrows, "bound": "tensor", "unit": "TFLOP/s", "peak": peak, "peak_source": kind, "shapes": shapes}


# ---------------------------------------------------------------------------------------
# the other configs of the metric, as compact extra keys of the one-GPU line
# ---------------------------------------------------------------------------------------
def _graph_time_us(calls, reps=3):
    """Device time per call of a list of closures: warmed up and captured as ONE CUDA graph on a side stream (the calls
    rotate over weight sets larger than L2), replayed `reps` times between two CUDA events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            for fn in calls:
                fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for fn in calls:
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(reps):
            graph.replay()
        e1.record(side)
        torch.cuda.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))


def _entry(k, n, m, us, nbytes, hbm_peak, tensor_peak, **extra):
    """{shape, m, us, frac, bound}: frac against the roofline that bounds the call (the longer of bytes / HBM peak
    and flops / tensor peak)."""
    t_hbm = nbytes / (hbm_peak * 1e3)                   # us
    t_tc = 2.0 * m * n * k / (tensor_peak * 1e6)         # us
    e = {"shape": [k, n], "m": m, "us": round(us, 2), "bound": "hbm" if t_hbm >= t_tc else "tensor",
         "frac": round(max(t_hbm, t_tc) / us, 4)}
    e.update(extra)
    return e


def extra_configs(dev):
    """cfg1 (one 4096x4096 int4 linear), cfg2 (int8 per-channel, both routes), cfg3 (a Mistral-7B layer with act-order)
    and the prefill config at all its batch sizes and both dtypes.  Weight sets rotate (> 2x L2 per measurement)."""
    import minit_b200 as M
    hbm_peak, _ = peaks()
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    tensor_peak = float(json.load(open(path))["bf16_tflops"]) if os.path.exists(path) else 1590.0
    gen = torch.Generator(device=dev).manual_seed(321)
    out = {}

    def gptq(k, n, dtype=torch.float16):
        qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        sc = (0.002 + 0.018 * torch.rand((k // GROUP, n), device=dev, generator=gen)).to(dtype)
        return qw, qz, sc

    def nsets(nbytes):
        return max(2, min(40, int(300e6 // nbytes) + 1))

    # ---- cfg1 ----
    k = n = 4096
    sets = [gptq(k, n) for _ in range(nsets(weight_bytes(k, n)))]
    rows = []
    for m in (1, 16):
        x = torch.randn((m, k), device=dev, generator=gen).half()
        o = torch.empty((m, n), device=dev, dtype=torch.float16)
        calls = [(lambda s=s_: M.quantized_matrix_multiply(x, s[0], s[1], s[2], None, bits=4, out=o, flags=4)) for s_ in sets]
        rows.append(_entry(k, n, m, _graph_time_us(calls), algorithmic_bytes(m, k, n), hbm_peak, tensor_peak))
    out["cfg1_int4_4096"] = rows
    del sets

    # ---- cfg2: int8, one scale per output channel; plain [K,N] layout and packed once into the 8-bit word layout ----
    rows = []
    for k, n in ((4096, 4096), (4096, 11008), (11008, 4096)):
        cnt = nsets(k * n)
        ws = [torch.randint(-127, 128, (k, n), device=dev, dtype=torch.int32, generator=gen).to(torch.int8) for _ in range(cnt)]
        scs = [(0.001 + 0.009 * torch.rand((n,), device=dev, generator=gen)).half() for _ in range(cnt)]
        packed = [M.pack_w8(w) for w in ws]
        for m in (1, 8, 32, 128, 512):
            x = torch.randn((m, k), device=dev, generator=gen).half()
            o = torch.empty((m, n), device=dev, dtype=torch.float16)
            nb = k * n + 2 * n + 2 * m * k + 2 * m * n
            plain = [(lambda w=w_, sc=sc_: M.w8_perchannel_matrix_multiply(x, w, sc, out=o)) for w_, sc_ in zip(ws, scs)]
            pk = [(lambda q=q_, sc=sc_: M.quantized_matrix_multiply(x, q, None, sc.view(1, -1), None, bits=8, out=o)) for q_, sc_ in zip(packed, scs)]
            rows.append(_entry(k, n, m, _graph_time_us(pk), nb, hbm_peak, tensor_peak, route="packed (mt_w8_pack + mt_qgemm)",
                               us_plain_layout=round(_graph_time_us(plain), 2)))
        del ws, scs, packed
    out["cfg2_int8_perchannel"] = rows

    # ---- cfg3: the seven linears of a Mistral-7B layer, act-order g_idx, rows sorted by group once at load ----
    lin = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336), ("up", 4096, 14336),
           ("down", 14336, 4096)]
    layers = []
    for _ in range(3):
        layer = []
        for _, k, n in lin:
            qw, qz, sc = gptq(k, n)
            g_idx = (torch.arange(k, device=dev) // GROUP)[torch.randperm(k, device=dev, generator=gen)].to(torch.int32)
            qs, perm = M.sort_act_order(qw, g_idx, k // GROUP, 4)
            layer.append((qs, qz, sc, perm))
            del qw
        layers.append(layer)
    rows = []
    for m in (1, 4, 16, 64):
        xs = {k: torch.randn((m, k), device=dev, generator=gen).half() for k in (4096, 14336)}
        os_ = {n: torch.empty((m, n), device=dev, dtype=torch.float16) for n in (4096, 1024, 14336)}
        calls = []
        for layer in layers:
            for (_, k, n), (qs, qz, sc, perm) in zip(lin, layer):
                calls.append(lambda qs=qs, qz=qz, sc=sc, perm=perm, k=k, n=n: M.quantized_matrix_multiply_ordered(xs[k], qs, qz, sc, perm, bits=4, out=os_[n]))
        us_layer = _graph_time_us(calls) * len(lin)
        nb = sum(algorithmic_bytes(m, k, n) + 4 * k for _, k, n in lin)
        rows.append({"m": m, "us_per_layer": round(us_layer, 2), "bound": "hbm", "frac": round(nb / (hbm_peak * 1e3) / us_layer, 4),
                     "launches_per_layer": len(lin) if m <= 2 else 2 * len(lin)})
    out["cfg3_mistral7b_layer_actorder"] = rows
    del layers

    # ---- cfg5: prefill, every batch size and both dtypes ----
    rows = []
    for dtype, name in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        for k, n in ((4096, 6144), (4096, 28672), (14336, 4096)):
            sets = [gptq(k, n, dtype) for _ in range(2)]
            for m in (2048, 4096, 8192):
                x = torch.randn((m, k), device=dev, generator=gen).to(dtype)
                o = torch.empty((m, n), device=dev, dtype=dtype)
                for i in range(2):
                    M.quantized_matrix_multiply(x, *sets[i % 2], None, bits=4, out=o)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(4):
                    M.quantized_matrix_multiply(x, *sets[i % 2], None, bits=4, out=o)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / 4
                rows.append(_entry(k, n, m, us, algorithmic_bytes(m, k, n), hbm_peak, tensor_peak, dtype=name,
                                   tflops=round(2.0 * m * n * k / us / 1e6, 1)))
                del x, o
            del sets
    out["cfg5_prefill"] = rows
    out["note"] = ("CUDA-graph loops over weight sets in rotation (> 2x L2), device time per call; frac is against the measured HBM "
                   "peak (%.0f GB/s) or the measured dense bf16 burst peak (%.0f TFLOP/s), whichever bounds the call" % (hbm_peak, tensor_peak))
    return out


def parity_check(world, rank, dev, far, comm, ms=(1, 8)):
    """Outside the timed region, at every N: one row-parallel linear of each kind (o, down) of the workload at
    M = 1 and M = 8 through the same call the timed step makes (the fused GEMM + all-reduce, the NCCL all-reduce
    after the GEMM, or the plain GEMM on one GPU), on seeded UNSHARDED weights that every rank generates
    identically on the host and slices on K by rank (minit/collective/dispatch.py:33-37,
    minit/collective/tensor.py:72-73).  A 512-column slice of every rank's output is compared with the oracle's
    dequantize-then-matmul of the unsharded weight (max |err| <= 1e-2 * rms, the test suite's bound), and the
    outputs of all ranks must be bit-identical.  The oracle is only the checker here."""
    import torch.distributed as dist
    import minit_b200 as M
    from minit_b200.collective.quantized import shard_gptq_row
    from oracle import qlinear_oracle as O
    cols = slice(1024, 1536)
    res = {"cases": [], "ok": True, "bound": "max|out - ref| <= 1e-2 * rms(ref) on 512 columns; outputs identical on all ranks"}
    for name, k, n in (("o", HIDDEN, HIDDEN), ("down", INTER, HIDDEN)):
        gen = torch.Generator().manual_seed(4242 + k)
        g = k // GROUP
        qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=gen, dtype=torch.int64).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (g, n // 8), generator=gen, dtype=torch.int64).to(torch.int32)
        sc = (0.002 + 0.018 * torch.rand((g, n), generator=gen)).half()
        w_ref = O.dequantize_packed(qw[:, cols].contiguous(), None, qz[:, cols.start // 8:cols.stop // 8].contiguous(),
                                    sc[:, cols].contiguous(), BITS)
        sqw, sqz, ssc, _ = shard_gptq_row(qw, qz, sc, BITS, rank, world)
        sqw, sqz, ssc = sqw.to(dev), sqz.to(dev), ssc.to(dev)
        # (rows, flags): the dispatch's own choice at 1 and 8 rows, and at 8 rows the integer tensor-core kernel by flag (its
        # own exchange code in its epilogue)
        from minit_b200 import _lib
        cases = [(m, 0) for m in ms] + ([(8, _lib.FLAG_FORCE_MID)] if world > 1 and far is not None else [])
        for m, case_flags in cases:
            x = torch.randn((m, k), generator=gen).half()
            ref = O.qlinear(x, w_ref)
            xs = x[:, k // world * rank:k // world * (rank + 1)].contiguous().to(dev)
            if world > 1 and far is not None:
                out = far.matmul(xs, sqw, sqz, ssc, None, bits=BITS, flags=case_flags)
            else:
                out = M.quantized_matrix_multiply(xs, sqw, sqz, ssc, None, bits=BITS)
                if world > 1:
                    from minit_b200.nccl.dispatch import all_reduce_
                    all_reduce_(comm.version, out)
            torch.cuda.synchronize()
            ok, err, bound = O.tolerance_ok(out[:, cols], ref, 1e-2)
            same = True
            if world > 1:
                gathered = [torch.empty_like(out) for _ in range(world)]
                dist.all_gather(gathered, out)
                same = all(torch.equal(gathered[0], t) for t in gathered[1:])
                flag = torch.tensor([0 if (ok and same) else 1], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                ok = ok and int(flag.item()) == 0
            res["cases"].append({"linear": name, "k": k, "n": n, "m": m, "max_err": err, "bound": bound, "ranks_identical": same,
                                 "kernel": "integer tensor-core (by flag)" if case_flags else "dispatch"})
            res["ok"] = res["ok"] and ok and same
        del sqw, sqz, ssc
    return res


def error_words():
    """Non-zero error words of this process's workspaces: a bounded wait inside a kernel expired."""
    from minit_b200 import _lib
    torch.cuda.synchronize()
    return [w for w in (_lib.workspace_error_word(ws) for ws in _lib._workspaces.values()) if w != 0]


def run_ours(args):
    import torch.distributed as dist
    import minit_b200 as M
    from minit_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    far = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from minit_b200.distributed import DistributedCommunicator, initialize_world
        from minit_b200.nccl import NCCLTensor
        from minit_b200.nccl.library import exchange_unique_id
        from minit_b200.nccl.dispatch import all_reduce_
        initialize_world(rank, world)
        uid = exchange_unique_id(rank)
        version = NCCLTensor.connect(uid, rank, world, device=local_rank)
        comm = DistributedCommunicator(version)
        if args.allreduce == "fused":
            from minit_b200.collective import FusedAllReduce
            far = FusedAllReduce(m_max=max(16, args.m), n_max=HIDDEN)

    m = args.m
    shapes = layer_shapes(args.shard_as if (world == 1 and args.shard_as > 1) else world)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    layers = []
    for _ in range(args.layers):
        lin = []
        for name, k, n, kind in shapes:
            qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
            qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
            sc = (0.002 + 0.018 * torch.rand((k // GROUP, n), device=dev, generator=gen)).half()
            lin.append((qw, qz, sc))
        layers.append(lin)
    # synthetic activations, one per distinct input width (N(0,1)); pinned host copies feed the e2e run
    xs_host = [torch.randn((m, k), generator=torch.Generator().manual_seed(7 + i)).half().pin_memory()
               for i, (_, k, _, _) in enumerate(shapes)]
    xs = [x.to(dev) for x in xs_host]
    outs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _, _, n, _ in shapes]
    out_host = torch.empty((m, HIDDEN), dtype=torch.float16).pin_memory()
    flags = _lib.FLAG_PDL if args.pdl else 0
    flags |= {"auto": 0, "one": _lib.FLAG_AR_ONE_SHOT, "two": _lib.FLAG_AR_TWO_SHOT}[args.ar_mode]

    # decode (M <= 2): the linears of `--chain` consecutive layers go to ONE resident launch (mt_qgemm_chain); every
    # entry waits for the one before it, as the stream order of separate launches would make it
    chains = []
    chain_layers = max(0, min(args.chain, 4)) if m <= 2 else 0
    if chain_layers:
        from minit_b200.chain import ChainEntry, LinearChain
        for l0 in range(0, len(layers), chain_layers):
            entries = []
            for lin in layers[l0:l0 + chain_layers]:
                for i, (qw, qz, sc) in enumerate(lin):
                    entries.append(ChainEntry(xs[i], qw, qz, sc, outs[i], allreduce=(far is not None and shapes[i][3] == "row")))
            chains.append(LinearChain(entries, bits=BITS, fused=far, flags=args.chain_flags))
        if comm is not None and far is None:
            chains = []                                   # NCCL all-reduce between the linears: separate launches
    launches_per_step = len(chains) if chains else args.layers * len(shapes)

    def one_pass():
        if chains:
            for c in chains:
                c()
            return
        for lin in layers:
            for i, (qw, qz, sc) in enumerate(lin):
                if comm is not None and shapes[i][3] == "row" and far is not None:
                    far.matmul(xs[i], qw, qz, sc, None, bits=BITS, out=outs[i], flags=flags)   # GEMM + all-reduce, one kernel
                    continue
                M.quantized_matrix_multiply(xs[i], qw, qz, sc, None, bits=BITS, out=outs[i], flags=flags)
                if comm is not None and shapes[i][3] == "row":
                    all_reduce_(comm.version, outs[i])

    def one_pass_e2e():
        for x, xh in zip(xs, xs_host):
            x.copy_(xh, non_blocking=True)
        one_pass()
        out_host.copy_(outs[3], non_blocking=True)

    def make_runner(fn):
        if args.no_graph:
            return fn, "eager"
        try:
            fn(); torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g.replay, "cuda_graph"
        except Exception as e:  # noqa: BLE001  graph capture is an optimisation, eager is the same work
            torch.cuda.synchronize()
            if rank == 0:
                print(f"[bench] graph capture unavailable ({type(e).__name__}); running eager", file=sys.stderr)
            return fn, "eager"

    def timed(fn, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        clocks = sampler.stop() if sampler else None
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, clocks

    runner, mode = make_runner(one_pass)
    ms_step, clocks = timed(runner, args.steps, args.warmup, sample_clocks=True)
    e2e_runner, e2e_mode = make_runner(one_pass_e2e)
    ms_e2e, _ = timed(e2e_runner, args.steps, args.warmup)
    # the same end-to-end step without the CUDA graph: one eager call of the Python wrapper per linear, which is the
    # seam the reference has (examples/qwen1_5_int8.py:244-267); its per-call host cost shows here
    ms_e2e_eager = None
    if mode == "cuda_graph" and not args.no_extra:
        ms_e2e_eager, _ = timed(one_pass_e2e, 5, 2)

    # where the step's time goes at N > 1: the same per-rank linears with no exchange at all, and the exchange on a
    # GEMV so small ([1,128] x [128,8192]) that the difference to the same GEMV alone is the mailbox hand-over itself
    # (peer stores + bounded poll + the skew between the ranks)
    ar_split = None
    if world > 1 and far is not None and not args.no_extra:
        def local_pass():
            for lin in layers:
                for i, (qw, qz, sc) in enumerate(lin):
                    M.quantized_matrix_multiply(xs[i], qw, qz, sc, None, bits=BITS, out=outs[i], flags=flags)
        r_local, _ = make_runner(local_pass)
        ms_local, _ = timed(r_local, max(3, args.steps // 2), 3)
        tiny = []
        for _ in range(2):
            tiny.append((torch.randint(-2**31, 2**31 - 1, (128 // 8, HIDDEN), device=dev, dtype=torch.int64, generator=gen).to(torch.int32),
                         torch.randint(-2**31, 2**31 - 1, (1, HIDDEN // 8), device=dev, dtype=torch.int64, generator=gen).to(torch.int32),
                         (0.002 + 0.018 * torch.rand((1, HIDDEN), device=dev, generator=gen)).half()))
        xt = torch.randn((m, 128), device=dev).half()
        ot = torch.empty((m, HIDDEN), dtype=torch.float16, device=dev)

        def tiny_fused():
            for i in range(40):
                far.matmul(xt, *tiny[i & 1], None, bits=BITS, out=ot, flags=flags)

        def tiny_local():
            for i in range(40):
                M.quantized_matrix_multiply(xt, *tiny[i & 1], None, bits=BITS, out=ot, flags=flags)
        r_f, _ = make_runner(tiny_fused)
        r_l, _ = make_runner(tiny_local)
        ms_f, _ = timed(r_f, 10, 3)
        ms_l, _ = timed(r_l, 10, 3)
        ar_split = {"ms_per_step_no_exchange": ms_local, "exchanges_per_step": 2 * args.layers,
                    "gemv_128x8192_us": ms_l * 1e3 / 40, "gemv_128x8192_allreduce_us": ms_f * 1e3 / 40,
                    "exchange_us": (ms_f - ms_l) * 1e3 / 40}

    # correctness evidence beside the timing, at every N: no bounded wait expired during the timed steps, and the
    # row-parallel linears (with their all-reduce) reproduce the oracle on unsharded weights
    words_timed = error_words()
    parity = parity_check(world, rank, dev, far, comm)
    parity["error_words_after_timed_steps"] = words_timed
    bad_words = words_timed + error_words()
    if world > 1:
        t = torch.tensor([len(bad_words)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity["error_word_any_rank"] = int(t.item())
        parity["ok"] = parity["ok"] and int(t.item()) == 0
    else:
        parity["ok"] = parity["ok"] and not bad_words

    per_rank_wbytes = args.layers * sum(weight_bytes(k, n) for _, k, n, _ in shapes)
    per_rank_abytes = args.layers * sum(algorithmic_bytes(m, k, n) for _, k, n, _ in shapes)
    total_wbytes = per_rank_wbytes * world
    hbm_peak, peak_kind = peaks()
    linears_per_step = args.layers * len(shapes)
    if chains and not all(c.single_launch for c in chains):
        raise SystemExit("the library declined the chain launch; rerun with --chain 0")
    achieved = per_rank_abytes / (ms_step * 1e-3) / 1e9     # per GPU: bytes of its launches / time of its launches
    # DRAM bytes per launch of the decode GEMV: ncu measured 245.85 MB read + 3.77 MB written for
    # 244.2 MB of algorithmic bytes on gate/up, 122.12 + 3.41 MB for 122.1 MB on down
    # (profiles/qgemm_vstream_8192x57344_m1.md, profiles/qgemm_vec_split_28672x8192_m1.md); traffic
    # scales with the bytes.
    traffic = 1.025 * per_rank_abytes / launches_per_step
    launch_desc = ("chain: %d linears (%d layers) per launch" % (chain_layers * len(shapes), chain_layers)) if chains else "one launch per linear"
    line = {
        "metric": "int4 dequant-GEMM weight GB/s at M=%d" % m, "value": total_wbytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 (int4 weights, f32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"llama3-70b-gptq-int4-g128-decode-linears-tp{world}", "m": m, "layers": args.layers,
                   "linears_per_layer": [[n_, k_, nn_] for n_, k_, nn_, _ in shapes], "launch": mode, "launches_per_step": launches_per_step, "kernel_launch": launch_desc, "pdl": bool(args.pdl), "allreduce": (args.allreduce if world > 1 else "none"),
                   "l2": "inputs larger than L2 (%.1f GB of weights per rank per step)" % (per_rank_wbytes / 1e9),
                   "tokens_per_s": m / (ms_step * 1e-3)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": traffic, "traffic_unit": "bytes per launch (average launch)", "peak_source": peak_kind,
                     "note": "per GPU, averaged over the %d launches of a step (algorithmic bytes / device time)" % launches_per_step},
        "e2e": {"value": total_wbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e, "launch": e2e_mode,
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in xs_host), "d2h_bytes_per_step": out_host.numel() * 2,
                "note": "weights stay resident (loaded once, like model parameters); activations cross PCIe every step"},
        "e2e_eager": None if ms_e2e_eager is None else {"value": total_wbytes / (ms_e2e_eager * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e_eager,
                                                          "launch": "eager: %d Python calls per step (%s)" % (launches_per_step, launch_desc)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "parity_check": parity,
    }
    if ar_split is not None:
        line["allreduce_split"] = ar_split
    if rank == 0 and world == 1 and m == 1 and not args.no_prefill:
        line["prefill_m4096"] = prefill_m4096(dev)
    if rank == 0 and world == 1 and m == 1 and not args.no_extra:
        line["other_configs"] = extra_configs(dev)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    if not parity["ok"]:
        raise SystemExit("parity check failed: " + json.dumps(parity))


# ---------------------------------------------------------------------------------------
# CPU arm: the oracle port (reference dequantize-then-matmul restated with torch on host cores)
# ---------------------------------------------------------------------------------------
def _cpu_sample(n_cols: int, m: int = 1, seed: int = 0):
    from oracle import qlinear_oracle as O
    gen = torch.Generator().manual_seed(seed)
    k = HIDDEN
    qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n_cols), generator=gen, dtype=torch.int64).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n_cols // 8), generator=gen, dtype=torch.int64).to(torch.int32)
    sc = (0.002 + 0.018 * torch.rand((k // GROUP, n_cols), generator=gen)).half()
    x = torch.randn((m, k), generator=gen).half()

    def run():
        w = O.dequantize_packed(qw, None, qz, sc, BITS)
        return O.qlinear(x, w)
    return run, weight_bytes(k, n_cols)


def cpu_baseline(budget_s: float):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    run, nbytes = _cpu_sample(1024)
    run()
    t0 = time.perf_counter(); run(); dt = time.perf_counter() - t0
    cols = int(max(1024, min(57344, (budget_s / 3 / max(dt, 1e-4)) * 1024)) // 1024 * 1024)
    run, nbytes = _cpu_sample(cols)
    run()
    ts = []
    for _ in range(2):
        t0 = time.perf_counter(); run(); ts.append(time.perf_counter() - t0)
    dt = statistics.median(ts)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"dequantize-then-matmul (torch, fp32 accumulate) of one int4 g128 linear K=8192 N={cols} at M=1, "
                      f"median of 2 runs of {dt:.2f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    total = args.steps + args.warmup
    run, _ = _cpu_sample(1024, args.m)
    run()
    t0 = time.perf_counter(); run(); dt = time.perf_counter() - t0
    per_step = min(10.0, 150.0 / max(total, 1))
    cols = int(max(1024, min(57344, (per_step / max(dt, 1e-4)) * 1024)) // 1024 * 1024)
    run, nbytes = _cpu_sample(cols, args.m)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    value = nbytes / dt / 1e9
    sample = (f"each step = dequantize-then-matmul (oracle port of minit/quantize/dispatch.py:14-20 + fp32-accumulate matmul, "
              f"torch on host cores) of one int4 g128 linear K=8192 N={cols} at M={args.m}")
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    print(json.dumps({
        "impl": "reference", "metric": "int4 dequant-GEMM weight GB/s at M=%d" % args.m, "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 (int4 weights, f32 accumulate)", "data": "synthetic",
        "config": {"workload": f"llama3-70b-gptq-int4-g128-decode-linears-tp{world}", "m": args.m},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_single_shape(args):
    """One linear, a few launches: the command the ncu captures under profiles/ were taken with.
    Prints device time and the roofline of that one kernel."""
    import minit_b200 as M
    k, n = (int(v) for v in args.single_shape.split(","))
    m, bits = args.m, args.bits
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    pack = 32 // bits
    gen = torch.Generator(device=dev).manual_seed(0)
    dtype = torch.bfloat16 if args.bf16 else torch.float16
    copies = max(2, min(16, int(400e6 // weight_bytes(k, n, bits)) + 1))   # rotate weight sets: HBM, not L2
    sets = []
    for _ in range(copies):
        qw = torch.randint(-2**31, 2**31 - 1, (k // pack, n), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // pack), device=dev, dtype=torch.int64, generator=gen).to(torch.int32)
        sc = (0.002 + 0.018 * torch.rand((k // GROUP, n), device=dev, generator=gen)).to(dtype)
        sets.append((qw, qz, sc))
    x = torch.randn((m, k), device=dev, dtype=torch.float32).to(dtype)
    out = torch.empty((m, n), device=dev, dtype=dtype)
    flags = {"auto": 0, "ring": 1, "tc": 2, "vec": 16, "umma": 32, "mid": 128, "tcx": 258, "tcw": 514}[args.kernel] | ((args.tune & 0x1f) << 24) | (4 if args.pdl and args.kernel in ("auto", "ring", "vec") else 0)

    def one():
        for qw, qz, sc in sets:
            M.quantized_matrix_multiply(x, qw, qz, sc, None, bits=bits, out=out, flags=flags)
    if args.no_graph:
        for _ in range(args.warmup):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.steps * copies)
    else:
        us = _graph_time_us([one], reps=max(1, args.steps)) / copies
    hbm_peak, kind = peaks()
    ab = k * n * bits // 8 + (k // GROUP) * n * 2 + (k // GROUP) * n * bits // 8 + 2 * m * k + 2 * m * n
    line = {"single_shape": [k, n], "m": m, "bits": bits, "kernel": args.kernel, "us_per_launch": us,
            "weight_GBps": weight_bytes(k, n, bits) / us / 1e3, "TFLOPs": 2.0 * m * n * k / us / 1e6,
            "hbm_frac": ab / us / 1e3 / hbm_peak, "launch": "%s, %d weight sets in rotation" % ("eager" if args.no_graph else "cuda graph", copies)}
    ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(ppath):
        line["tensor_frac_of_burst"] = line["TFLOPs"] / float(json.load(open(ppath))["bf16_tflops"])
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", "--m", dest="m", type=int, default=1, help="decode batch M (use --batch under torchrun)")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--chain", type=int, default=0, help="decode: layers per resident launch of mt_qgemm_chain (0: one launch per linear, which measures faster)")
    ap.add_argument("--tune", type=int, default=0, help="--single-shape: tuning bits 24-28 of the flags")
    ap.add_argument("--ar-mode", default="auto", choices=["auto", "one", "two"],
                    help="fused all-reduce of 3..32 rows: one-shot, two-shot (partials to the column's owner, the sum back) or the library's default (one-shot)")
    ap.add_argument("--chain-flags", type=int, default=0, help="tuning bits passed to the chain launch")
    ap.add_argument("--shard-as", type=int, default=1, help="one GPU only: time the per-rank shapes of an N-way split, no exchange")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="row-parallel exchange: fused into the GEMM epilogue over peer memory, or an NCCL all-reduce after it")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the M = 4096 TFLOP/s measurement of the default one-GPU run")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configs (cfg1, cfg2 int8, cfg3 act-order, all prefill sizes) and the eager e2e figure")
    ap.add_argument("--single-shape", default=None, help="K,N : time one linear instead of the workload (profiling aid)")
    ap.add_argument("--mlp-block", action="store_true", help="time the feed-forward block with separate and with fused elementwise steps")
    ap.add_argument("--decode-layer", action="store_true", help="time whole decoder layers (norms, rope, attention, fused linears) for one token")
    ap.add_argument("--attention", action="store_true", help="time decode attention alone over --context cached positions")
    ap.add_argument("--context", type=int, default=4096, help="--decode-layer: cached positions")
    ap.add_argument("--kernel", default="auto", choices=["auto", "ring", "tc", "vec", "umma", "mid", "tcx", "tcw"])
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--bf16", action="store_true")
    args = ap.parse_args()
    if args.single_shape:
        return run_single_shape(args)
    if args.mlp_block:
        return run_mlp_block(args)
    if args.decode_layer:
        return run_decode_layer(args)
    if args.attention:
        return run_attention(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
