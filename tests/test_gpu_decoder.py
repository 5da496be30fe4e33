"""Parity of the decoder-layer steps around the linears (RMSNorm, rotary embedding + cache append, decode
attention) and of the whole layer with the oracle's restatement of the reference, through the C ABI.

Tolerances: RMSNorm and the rotary embedding evaluate the reference's fp32 expression and round once, so they
agree with the oracle to one ulp of the result (summation order, fused multiply-add).  Attention is computed
in fp32 and rounded once where the reference rounds scores, scaled scores, probabilities and output to the
tensor dtype; it is compared with an fp32 evaluation (tight) and with the stepwise oracle (the north-star GEMM
bound, 1e-2 * rms).
"""
import math

import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def D(lib_built):
    from minit_b200 import decoder
    return decoder


def ulp_of(v, dtype):
    bits = 10 if dtype == torch.float16 else 7
    return torch.exp2(torch.floor(torch.log2(v.abs().clamp_min(2.0 ** -14))) - bits)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,h", [(1, 8192), (3, 4096), (16, 512), (1, 8), (130, 5120)])
def test_rms_norm(D, dtype, rows, h):
    gen = torch.Generator().manual_seed(rows + h)
    x = (torch.randn((rows, h), generator=gen) * 3).to(dtype)
    w = (1 + 0.2 * torch.randn((h,), generator=gen)).to(dtype)
    out = D.rms_norm(x.to(DEV), w.to(DEV), 1e-5).cpu()
    ref = O.rms_norm(x, w, 1e-5)
    assert ((out.float() - ref.float()).abs() <= ulp_of(ref.float(), dtype)).all()
    assert (out == ref).float().mean() > 0.98          # the odd element differs by the summation order


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,hq,hkv,offset,d", [(1, 64, 8, 0, 128), (1, 64, 8, 777, 128), (5, 32, 8, 19, 128), (3, 8, 8, 1000, 128), (2, 4, 1, 7, 128),
                                               (4, 8, 2, 11, 64), (2, 6, 3, 300, 96), (40, 4, 4, 0, 256)])
def test_rope_append(D, dtype, m, hq, hkv, offset, d):
    gen = torch.Generator().manual_seed(m + hq + offset)
    qkv = torch.randn((m, (hq + 2 * hkv) * d), generator=gen).to(dtype)
    cos, sin = O.rope_tables(d, 1024, 5e5, dtype)
    cache = D.KVCache(1024, hkv, d, dtype, DEV)
    sentinel = torch.full_like(cache.k, 7.0)
    cache.k.copy_(sentinel); cache.v.copy_(sentinel)
    q = D.rope_append(qkv.to(DEV), cos.to(DEV), sin.to(DEV), cache, hq, offset).cpu()
    x = qkv.reshape(m, hq + 2 * hkv, d)
    q_ref = O.rope(x[:, :hq], cos, sin, offset)
    k_ref = O.rope(x[:, hq:hq + hkv], cos, sin, offset)
    close = lambda a, b: ((a.float() - b.float()).abs() <= ulp_of(b.float(), dtype)).all()
    assert close(q, q_ref)
    assert close(cache.k[offset:offset + m].cpu(), k_ref)
    assert torch.equal(cache.v[offset:offset + m].cpu(), x[:, hq + hkv:])                 # v is a copy
    # nothing else in the cache was touched
    assert (cache.k[:offset] == 7).all() and (cache.k[offset + m:] == 7).all()
    assert (cache.v[:offset] == 7).all() and (cache.v[offset + m:] == 7).all()
    # the tables of the host module are the oracle's
    c2, s2 = D.rope_tables(d, 1024, 5e5, dtype, DEV)
    assert torch.equal(c2.cpu(), cos) and torch.equal(s2.cpu(), sin)


@pytest.mark.parametrize("variant", [0, 1 << 24, 2 << 24], ids=["auto", "split", "stream"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,hq,hkv,offset,bias", [(1, 8, 2, 0, False), (1, 16, 4, 300, True), (2, 8, 2, 41, False), (3, 8, 2, 7, True)])
def test_qkv_linear_with_rope_epilogue(D, variant, dtype, m, hq, hkv, offset, bias):
    """The fused q/k/v linear with rotary embedding + cache append as its epilogue, against the oracle's linear followed
    by its rope; M = 3 takes the two-launch path (GEMM into scratch, then mt_rope_append)."""
    d, k, bits = 128, 1024, 4
    n = (hq + 2 * hkv) * d
    c = O.make_gptq_case(k, n, m, bits=bits, dtype=dtype, seed=hq + offset + m, bias=bias, scale_lo=0.001, scale_hi=0.004)
    cos, sin = O.rope_tables(d, 512, 5e5, dtype)
    cache = D.KVCache(512, hkv, d, dtype, DEV)
    cache.k.fill_(7.0); cache.v.fill_(7.0)
    dv = lambda t: t.to(DEV)
    q = D.qkv_rope_append(dv(c["x"]), dv(c["qweight"]), dv(c["qzeros"]), dv(c["scales"]), dv(cos), dv(sin), cache, hq, offset,
                          bits=bits, bias=dv(c["bias"]) if bias else None, flags=variant).cpu()
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], bits)
    y = O.qlinear(c["x"], w, c["bias"] if bias else None).reshape(m, hq + 2 * hkv, d)
    assert_close(q.reshape(m, -1), O.rope(y[:, :hq], cos, sin, offset).reshape(m, -1), "q")
    assert_close(cache.k[offset:offset + m].cpu().reshape(m, -1), O.rope(y[:, hq:hq + hkv], cos, sin, offset).reshape(m, -1), "k")
    assert_close(cache.v[offset:offset + m].cpu().reshape(m, -1), y[:, hq + hkv:].reshape(m, -1), "v")
    assert (cache.k[:offset] == 7).all() and (cache.k[offset + m:] == 7).all()
    assert (cache.v[:offset] == 7).all() and (cache.v[offset + m:] == 7).all()


def attention_fp32(q, k, v, offset):
    s_len, hq, d = q.shape
    r = hq // k.shape[1]
    kk, vv = k.repeat_interleave(r, dim=1).double(), v.repeat_interleave(r, dim=1).double()
    qk = torch.einsum("snd,tnd->nst", q.double(), kk) / math.sqrt(d)
    for i in range(s_len):
        qk[:, i, offset + i + 1:] = -math.inf
    return torch.einsum("nst,tnd->snd", torch.softmax(qk, dim=-1), vv).reshape(s_len, hq * d)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,hq,hkv,offset", [(1, 64, 8, 0), (1, 64, 8, 5), (1, 64, 8, 127), (1, 64, 8, 128), (1, 64, 8, 1500),
                                             (1, 32, 8, 4095), (4, 64, 8, 300), (2, 8, 8, 40), (3, 4, 1, 257), (1, 16, 2, 9000),
                                             (1, 16, 2, 13000), (2, 8, 1, 40000)])    # beyond 12288: four-warp CTAs, several clusters
def test_attention_decode(D, dtype, m, hq, hkv, offset):
    d = 128
    gen = torch.Generator().manual_seed(m + hq + offset)
    total = offset + m
    q = torch.randn((m, hq, d), generator=gen).to(dtype)
    k = torch.randn((total, hkv, d), generator=gen).to(dtype)
    v = torch.randn((total, hkv, d), generator=gen).to(dtype)
    cache = D.KVCache(total + 37, hkv, d, dtype, DEV)
    cache.k[:total].copy_(k); cache.v[:total].copy_(v)
    cache.k[total:].fill_(float("nan")); cache.v[total:].fill_(float("nan"))        # rows past the sequence are never read
    out = D.attention_decode(q.to(DEV), cache, offset).cpu()
    exact = attention_fp32(q, k, v, offset)
    err = (out.double() - exact).abs()
    assert not torch.isnan(out).any()
    assert (err <= 2e-3 * exact.abs().max() + ulp_of(exact.float(), dtype).double()).all(), f"max err {err.max().item():.4g}"
    step = O.attention(q, k, v, offset)
    if dtype == torch.float16:
        assert_close(out, step, f"attention vs stepwise oracle {dtype} m={m} offset={offset}")
    else:
        # in bf16 the reference's own intermediate roundings (scores and probabilities to 8 significant bits) move its
        # result by a few percent of the rms; the fused result must be at least as close to the exact one as the oracle is
        dev_step = (step.double() - exact).abs().max().item()                    # 3-8 % of the rms on these cases
        assert err.max().item() <= dev_step + 1e-6
        e = (out.double() - step.double()).abs().max().item()
        assert e <= 2 * dev_step + 1e-6, f"attention vs stepwise oracle bf16 m={m} offset={offset}: {e:.4g} > {2 * dev_step:.4g}"
    # a second call gives the same bits (the workspace is left zeroed, the merge order is fixed)
    assert torch.equal(D.attention_decode(q.to(DEV), cache, offset).cpu(), out)


def test_attention_decode_with_the_offset_on_the_device(D):
    """A captured step is replayed as the sequence grows: the position comes from device memory."""
    d, hq, hkv, cap = 128, 16, 2, 700
    gen = torch.Generator().manual_seed(1)
    k = torch.randn((cap, hkv, d), generator=gen).half()
    v = torch.randn((cap, hkv, d), generator=gen).half()
    cache = D.KVCache(cap, hkv, d, torch.float16, DEV)
    cache.k.copy_(k); cache.v.copy_(v)
    q = torch.randn((1, hq, d), generator=gen).half()
    pos = torch.zeros(1, dtype=torch.int32, device=DEV)
    for offset in (0, 131, 699):
        pos.fill_(offset)
        out = D.attention_decode(q.to(DEV), cache, 0, offset_dev=pos).cpu()
        assert_close(out, O.attention(q, k[:offset + 1], v[:offset + 1], offset), f"device offset {offset}")


def load_layer(D, layer, cases, norms):
    for name, c in cases.items():
        for buf in ("qweight", "qzeros", "scales", "g_idx"):
            layer.update_buffer(f"{name}.{buf}", c[buf].to(DEV))
    layer.update_buffer("input_layernorm.weight", norms[0].to(DEV))
    layer.update_buffer("post_attention_layernorm.weight", norms[1].to(DEV))


@pytest.mark.parametrize("b,m,hq,hkv,d,offset", [(1, 64, 8, 2, 128, 0), (2, 33, 8, 8, 64, 5), (3, 7, 12, 4, 96, 100), (1, 300, 4, 1, 256, 0),
                                                 (2, 1, 24, 2, 128, 57), (1, 130, 8, 8, 32, 3), (2, 40, 16, 2, 160, 31)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_for_prefill_sized_and_multi_sequence_batches(D, dtype, b, m, hq, hkv, d, offset):
    """examples/llama3_70b.py:103-115 for several sequences, many new tokens, head sizes other than 128 and more than eight
    query heads per kv head: against an fp64 evaluation (tight) and the stepwise oracle (the north-star bound)."""
    gen = torch.Generator().manual_seed(b + m + hq + d + offset)
    total = offset + m
    cap = total + 5
    q = torch.randn((b, m, hq, d), generator=gen).to(dtype)
    k = torch.full((b, cap, hkv, d), float("nan"), dtype=dtype)                      # rows past the sequence are never read
    v = torch.full((b, cap, hkv, d), float("nan"), dtype=dtype)
    k[:, :total] = torch.randn((b, total, hkv, d), generator=gen).to(dtype)
    v[:, :total] = torch.randn((b, total, hkv, d), generator=gen).to(dtype)
    out = D.attention(q.to(DEV), k.to(DEV), v.to(DEV), offset).cpu()
    assert out.shape == (b, m, hq * d) and not torch.isnan(out).any()
    for s_ in range(b):
        exact = attention_fp32(q[s_], k[s_, :total], v[s_, :total], offset)
        err = (out[s_].double() - exact).abs()
        assert (err <= 2e-3 * exact.abs().max() + ulp_of(exact.float(), dtype).double()).all(), f"seq {s_}: max err {err.max().item():.4g}"
        step = O.attention(q[s_], k[s_, :total], v[s_, :total], offset)
        if dtype == torch.float16:
            assert_close(out[s_], step, f"attention vs stepwise oracle b={b} m={m} d={d}")
        else:
            dev_step = (step.double() - exact).abs().max().item()
            assert err.max().item() <= dev_step + 1e-6


def test_attention_with_one_offset_per_sequence(D):
    """A ragged batch: every sequence has its own number of cached positions (device array)."""
    dtype, b, m, hq, hkv, d = torch.float16, 3, 5, 8, 2, 64
    offs = [0, 17, 40]
    gen = torch.Generator().manual_seed(77)
    cap = max(offs) + m + 3
    q = torch.randn((b, m, hq, d), generator=gen).to(dtype)
    k = torch.randn((b, cap, hkv, d), generator=gen).to(dtype)
    v = torch.randn((b, cap, hkv, d), generator=gen).to(dtype)
    out = D.attention(q.to(DEV), k.to(DEV), v.to(DEV), offsets=torch.tensor(offs, dtype=torch.int32, device=DEV)).cpu()
    for s_, off in enumerate(offs):
        exact = attention_fp32(q[s_], k[s_, :off + m], v[s_, :off + m], off)
        err = (out[s_].double() - exact).abs()
        assert (err <= 2e-3 * exact.abs().max() + ulp_of(exact.float(), dtype).double()).all()


@pytest.mark.parametrize("m,offset", [(1, 0), (1, 200), (3, 64), (40, 0), (24, 10)])
def test_decoder_layer_matches_the_reference_composition(D, m, offset):
    """TransformerBlock.forward of the reference (examples/llama3_70b.py:158-162) restated with the oracle, against
    QDecoderLayer: RMSNorm -> q/k/v -> rope -> cache -> attention -> o_proj + x -> RMSNorm -> feed-forward + h."""
    hidden, hq, r, d, inner, bits = 1024, 8, 4, 128, 2048, 4
    hkv = hq // r
    shapes = {"self_attn.q_proj": (hidden, hq * d), "self_attn.k_proj": (hidden, hkv * d), "self_attn.v_proj": (hidden, hkv * d),
              "self_attn.o_proj": (hq * d, hidden), "mlp.gate_proj": (hidden, inner), "mlp.up_proj": (hidden, inner),
              "mlp.down_proj": (inner, hidden)}
    cases = {n: O.make_gptq_case(k, nn, 1, bits=bits, seed=10 + i, scale_lo=0.001, scale_hi=0.004)
             for i, (n, (k, nn)) in enumerate(shapes.items())}
    gen = torch.Generator().manual_seed(99)
    norms = [(1 + 0.1 * torch.randn((hidden,), generator=gen)).half() for _ in range(2)]
    layer = D.QDecoderLayer(hidden, hq, r, d, inner, bits=bits)
    load_layer(D, layer, cases, norms)
    cos, sin = O.rope_tables(d, 512)
    total = offset + m
    k_hist = torch.randn((offset, hkv, d), generator=gen).half()
    v_hist = torch.randn((offset, hkv, d), generator=gen).half()
    cache = D.KVCache(512, hkv, d, torch.float16, DEV)
    cache.k[:offset].copy_(k_hist); cache.v[:offset].copy_(v_hist)
    x = torch.randn((m, hidden), generator=gen).half()
    out = layer(x.to(DEV), cache, cos.to(DEV), sin.to(DEV), offset).cpu()

    W = {n: O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], bits) for n, c in cases.items()}
    lin = lambda t, n: O.qlinear(t, W[n])
    xn = O.rms_norm(x, norms[0])
    q = O.rope(lin(xn, "self_attn.q_proj").reshape(m, hq, d), cos, sin, offset)
    k_new = O.rope(lin(xn, "self_attn.k_proj").reshape(m, hkv, d), cos, sin, offset)
    v_new = lin(xn, "self_attn.v_proj").reshape(m, hkv, d)
    a = O.attention(q, torch.cat([k_hist, k_new]), torch.cat([v_hist, v_new]), offset)
    h = O.add_residual(x, lin(a, "self_attn.o_proj"))
    hn = O.rms_norm(h, norms[1])
    ff = lin(O.swiglu(lin(hn, "mlp.gate_proj"), lin(hn, "mlp.up_proj")), "mlp.down_proj")
    ref = O.add_residual(h, ff)
    assert_close(out, ref, f"decoder layer m={m} offset={offset}")
    assert cache.length == total
    assert_close(cache.k[offset:total].cpu().reshape(m, -1), k_new.reshape(m, -1), "appended k")


def test_status_codes(D):
    from minit_b200 import _lib
    lib = _lib.lib
    z = torch.zeros(1 << 16, dtype=torch.int32, device=DEV)
    p = z.data_ptr()
    assert lib.mt_rms_norm(None, p, p, p, 1, 12, 1e-5, 0) == -3                     # H % 8
    assert lib.mt_rms_norm(None, p, p, p, 1, 16, 0.0, 0) == -3                      # eps
    assert lib.mt_rope_append(None, p, p, p, p, p, p, 1, 8, 2, 63, 0, None, 16, 16, 0) == -8      # odd head size
    assert lib.mt_attention(None, p, p, p, p, None, 1, 1, 8, 2, 80, 0, 8, 0.1, 0) == -8           # head size not a multiple of 32
    assert lib.mt_attention(None, p, p, p, p, None, 1, 4, 8, 3, 64, 0, 8, 0.1, 0) == -8           # 8 query heads over 3 kv heads
    assert lib.mt_attention(None, p, p, p, p, None, 1, 4, 8, 2, 64, 6, 8, 0.1, 0) == -3           # beyond the capacity
    assert lib.mt_rope_append(None, p, p, p, p, p, p, 4, 8, 2, 128, 14, None, 16, 64, 0) == -3    # beyond the capacity
    assert lib.mt_attention_decode(None, p, p, p, p, 1, 24, 2, 128, 0, None, 8, 0.1, p, 1 << 18, 0) == -8   # 12 query heads per kv head
    assert lib.mt_attention_decode(None, p, p, p, p, 1, 8, 2, 128, 0, None, 8, 0.1, p, 16, 0) == -6         # workspace too small
    assert lib.mt_attention_workspace_bytes(1, 8, 4096) > 0
    assert lib.mt_qgemm_rope_append(None, p, p, p, p, None, p, p, p, p, p, None, 1, 8, 2, 63, 256, 2, 4, 0, 0, None, 16, 16, p, 1 << 18, 0) == -8
    assert lib.mt_qgemm_rope_append(None, p, p, p, p, None, p, p, p, p, p, None, 1, 8, 2, 64, 256, 2, 4, 0, 0, None, 16, 16, p, 1 << 18, 0) == -1   # other head sizes go through scratch
    assert lib.mt_qgemm_rope_append(None, p, p, p, p, None, p, p, p, p, p, None, 4, 8, 2, 128, 256, 2, 4, 0, 0, None, 16, 16, p, 1 << 18, 0) == -1   # scratch at M > 2
