"""The CPU oracle against the committed golden vectors (outputs of the reference's own
dispatch_dequantize, see tests/golden/make_golden.py) and against hand-computed known answers."""
import os

import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dequant_golden.npz")
CASES = ["int4_f16", "int4_f16_act", "int4_bf16", "int4_f16_g32", "int8_f16", "int8_f16_act", "int8_bf16_act"]


def load_case(g, name):
    dt = torch.bfloat16 if int(g[f"{name}.is_bf16"]) else torch.float16
    scales = torch.from_numpy(g[f"{name}.scales_bits"]).view(dt)
    return dict(bits=int(g[f"{name}.bits"]), qweight=g[f"{name}.qweight"], qzeros=g[f"{name}.qzeros"],
                g_idx=g[f"{name}.g_idx"], scales=scales, w_bits=g[f"{name}.w_bits"])


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_dequantize_bit_exactly(name):
    c = load_case(np.load(GOLDEN), name)
    w = O.dequantize_packed(c["qweight"], c["g_idx"], c["qzeros"], c["scales"], c["bits"])
    assert np.array_equal(w.view(torch.int16).numpy(), c["w_bits"])


def test_oracle_w8_perchannel_is_the_one_group_special_case():
    g = np.load(GOLDEN)
    w_i8 = g["w8pc.w_i8"]
    scales = torch.from_numpy(g["w8pc.scales_bits"]).view(torch.float16)
    qweight, g_idx, qzeros, s = O.w8_perchannel_as_gptq(w_i8, scales)
    w = O.dequantize_packed(qweight, g_idx, qzeros, s, 8)
    assert np.array_equal(w.view(torch.int16).numpy(), g["w8pc.w_bits"])
    # and it equals w * scale rounded once
    direct = (torch.from_numpy(w_i8).float() * scales.float()).half()
    assert torch.equal(w, direct)


def test_known_answers():
    s = torch.tensor([[0.5, 0.25, 2.0, 1.0]], dtype=torch.float16)
    # 4-bit: q=0,z=15 -> (0-16)*s ; q=15,z=0 -> 14*s ; no wrap-around of z+1
    q = np.array([[0, 15, 0, 7]], dtype=np.uint8)
    z = np.array([[15, 0, 0, 7]], dtype=np.uint8)
    w = O.dequantize(q, np.zeros(1, np.int32), z, s)
    assert w.tolist() == [[-8.0, 3.5, -2.0, -1.0]]
    # 8-bit: q=255,z=255 -> -1*s ; per-channel midpoint z=127
    q = np.array([[255, 0, 128, 255]], dtype=np.uint8)
    z = np.array([[255, 255, 127, 0]], dtype=np.uint8)
    w = O.dequantize(q, np.zeros(1, np.int32), z, s)
    assert w.tolist() == [[-0.5, -64.0, 0.0, 254.0]]


@pytest.mark.parametrize("bits", [4, 8])
def test_pack_unpack_roundtrip_and_bit_positions(bits):
    rng = np.random.default_rng(bits)
    ps = 32 // bits
    q = rng.integers(0, 1 << bits, size=(4 * ps, 16), dtype=np.uint8)
    assert np.array_equal(O.unpack_rows(O.pack_rows(q, bits), bits), q)
    z = rng.integers(0, 1 << bits, size=(3, 2 * ps), dtype=np.uint8)
    assert np.array_equal(O.unpack_cols(O.pack_cols(z, bits), bits), z)
    # element k of a column sits at bits (k % pack) * bits of word k // pack (little-endian in the word)
    one = np.zeros((ps, 1), dtype=np.uint8)
    one[3, 0] = (1 << bits) - 1
    assert int(O.pack_rows(one, bits).view(np.uint32)[0, 0]) == ((1 << bits) - 1) << (3 * bits)
    onec = np.zeros((1, ps), dtype=np.uint8)
    onec[0, 2] = 1
    assert int(O.pack_cols(onec, bits).view(np.uint32)[0, 0]) == 1 << (2 * bits)


def test_int8_unpack_is_the_byte_view_the_reference_uses():
    # the reference's unpack reinterprets int32 as uint8 (examples/qwen1_5_int8.py:44): byte j of a word = element j
    rng = np.random.default_rng(0)
    qweight = rng.integers(-2**31, 2**31 - 1, size=(5, 7), dtype=np.int64).astype(np.int32)
    bytes_view = qweight.view(np.uint8).reshape(5, 7, 4).transpose(0, 2, 1).reshape(20, 7)
    assert np.array_equal(O.unpack_rows(qweight, 8), bytes_view)
    qzeros = rng.integers(-2**31, 2**31 - 1, size=(3, 6), dtype=np.int64).astype(np.int32)
    assert np.array_equal(O.unpack_cols(qzeros, 8), qzeros.view(np.uint8).reshape(3, 24))


def test_qlinear_fp32_accumulate_and_bias():
    c = O.make_gptq_case(256, 32, 3, bits=4, seed=5, bias=True)
    w = O.dequantize_packed(c["qweight"], c["g_idx"], c["qzeros"], c["scales"], 4)
    out = O.qlinear(c["x"], w, c["bias"])
    ref = (c["x"].double() @ w.double() + c["bias"].double())
    assert out.dtype == torch.float16
    assert (out.double() - ref).abs().max() <= 2e-3 * ref.abs().max()


def test_null_zeros_and_null_gidx_defaults():
    c = O.make_gptq_case(128, 16, 1, bits=4, group_size=64, seed=9)
    z = np.full((2, 16), 7, dtype=np.uint8)
    a = O.dequantize_packed(c["qweight"], None, None, c["scales"], 4)
    b = O.dequantize(O.unpack_rows(c["qweight"].numpy(), 4), np.arange(128) // 64, z, c["scales"])
    assert torch.equal(a, b)


@pytest.mark.parametrize("size", [2, 4])
def test_tensor_parallel_sharding_identities(size):
    c = O.make_gptq_case(512, 64, 4, bits=4, seed=11)
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4)
    full = c["x"].float() @ w.float()
    cols = []
    for r in range(size):
        qw, qz, s = O.shard_column(c["qweight"], c["qzeros"], c["scales"], 4, r, size)
        cols.append(c["x"].float() @ O.dequantize_packed(qw.contiguous(), None, qz.contiguous(), s.contiguous(), 4).float())
    assert torch.allclose(torch.cat(cols, dim=1), full, atol=1e-4)
    part = torch.zeros_like(full)
    ks = 512 // size
    for r in range(size):
        qw, qz, s = O.shard_row(c["qweight"], c["qzeros"], c["scales"], 4, r, size)
        wr = O.dequantize_packed(qw.contiguous(), None, qz.contiguous(), s.contiguous(), 4)
        part += c["x"][:, ks * r:ks * (r + 1)].float() @ wr.float()
    assert torch.allclose(part, full, atol=1e-3)


def test_elementwise_steps_of_the_feed_forward():
    """sigmoid / silu / swiglu / add_residual follow the reference's elementwise rules (one rounding per step)."""
    import numpy as np
    import torch
    from oracle import qlinear_oracle as O
    x = torch.tensor([-20.0, -3.0, -0.5, 0.0, 0.25, 2.0, 11.0]).half()
    s = O.sigmoid(x)
    assert s.dtype == torch.float16
    assert torch.equal(s, torch.sigmoid(x.double()).half())          # same value, rounded once
    assert torch.equal(O.silu(x), (x.double() * s.double()).half())
    u = torch.tensor([2.0, -1.0, 0.5, 3.0, -4.0, 1.5, 0.125]).half()
    assert torch.equal(O.swiglu(x, u), (O.silu(x).double() * u.double()).half())
    assert torch.equal(O.add_residual(x, u), (x.double() + u.double()).half())
    for dtype in (torch.float16, torch.bfloat16):
        g = (torch.randn(4096, generator=torch.Generator().manual_seed(0)) * 4).to(dtype)
        exact = torch.nn.functional.silu(g.double())
        ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
        assert ((O.silu(g).double() - exact).abs() <= exact.abs() * ulp * 1.5 + 2e-6).all()      # 2e-6: fp16 sigmoid is subnormal below g = -10


def test_gate_up_interleave_layout():
    """Blocks of eight output columns = four gate columns, then the four up columns of the same indices; packed
    zero points follow their columns."""
    import numpy as np
    from oracle import qlinear_oracle as O
    a = np.arange(2 * 16).reshape(2, 16)
    out = O.interleave_columns(a, a + 100)
    assert out[0].tolist() == [0, 1, 2, 3, 100, 101, 102, 103, 4, 5, 6, 7, 104, 105, 106, 107,
                               8, 9, 10, 11, 108, 109, 110, 111, 12, 13, 14, 15, 112, 113, 114, 115]
    for bits in (4, 8):
        g = O.make_gptq_case(256, 64, 1, bits=bits, seed=1)
        u = O.make_gptq_case(256, 64, 1, bits=bits, seed=2)
        qw, qz, sc = O.interleave_gate_up((g["qweight"], g["qzeros"], g["scales"].view(torch.int16)),
                                          (u["qweight"], u["qzeros"], u["scales"].view(torch.int16)), bits)
        # dequantizing the interleaved linear gives the interleaved dequantized weights
        w = O.dequantize_packed(torch.from_numpy(qw), None, torch.from_numpy(qz), torch.from_numpy(sc.view(np.int16)).view(torch.float16), bits)
        wg = O.dequantize_packed(g["qweight"], None, g["qzeros"], g["scales"], bits)
        wu = O.dequantize_packed(u["qweight"], None, u["qzeros"], u["scales"], bits)
        ref = O.interleave_columns(wg.view(torch.int16).numpy(), wu.view(torch.int16).numpy())
        assert np.array_equal(w.view(torch.int16).numpy(), ref)


def test_decoder_step_restatements():
    """rms_norm / rope / attention of the oracle: properties the reference's kernels have by construction (their CUDA
    sources cannot run without a GPU, so these restatements are pinned by properties, not by vectors)."""
    import math
    gen = torch.Generator().manual_seed(0)
    # rms_norm: unit weight gives rows of unit mean square; scaling the input leaves the output unchanged
    x = torch.randn((3, 256), generator=gen).half()
    y = O.rms_norm(x, torch.ones(256).half(), 1e-5).float()
    assert torch.allclose(y.pow(2).mean(dim=-1), torch.ones(3), atol=2e-3)
    assert torch.allclose(O.rms_norm(x * 4, torch.ones(256).half(), 1e-5).float(), y, atol=2e-3)
    # rope: position 0 is the identity, a rotation keeps the length of every (even, odd) pair
    cos, sin = O.rope_tables(128, 64)
    q = torch.randn((4, 2, 128), generator=gen).half()
    assert torch.equal(O.rope(q[:1], cos, sin, 0), q[:1])
    r = O.rope(q, cos, sin, 7).float().reshape(4, 2, 64, 2)
    assert torch.allclose(r.pow(2).sum(-1), q.float().reshape(4, 2, 64, 2).pow(2).sum(-1), atol=2e-2)
    # relative position: <rope(a, m), rope(b, n)> depends on m - n only
    a, b = q[:1, :1], q[1:2, :1]
    d1 = (O.rope(a, cos, sin, 5).float() * O.rope(b, cos, sin, 2).float()).sum()
    d2 = (O.rope(a, cos, sin, 25).float() * O.rope(b, cos, sin, 22).float()).sum()
    assert abs(d1 - d2) < 0.05 * (abs(d1) + 1)
    # attention: one cached position returns its v; causal: the first new token ignores the second
    k = torch.randn((6, 2, 128), generator=gen).half(); v = torch.randn((6, 2, 128), generator=gen).half()
    qq = torch.randn((2, 4, 128), generator=gen).half()
    one = O.attention(qq[:1], k[:1], v[:1], 0)
    assert torch.equal(one.reshape(4, 128)[0], v[0, 0]) and torch.equal(one.reshape(4, 128)[3], v[0, 1])   # heads 0-1 -> kv 0, 2-3 -> kv 1
    both = O.attention(qq, k, v, 4)
    first = O.attention(qq[:1], k[:5], v[:5], 4)
    assert torch.equal(both[0], first[0])
    ref = torch.softmax(torch.einsum("snd,tnd->nst", qq[1:].float(), k.repeat_interleave(2, 1).float()) / math.sqrt(128), -1)
    out = torch.einsum("nst,tnd->snd", ref, v.repeat_interleave(2, 1).float()).reshape(1, -1)
    assert torch.allclose(both[1:].float(), out, atol=2e-2)


@pytest.mark.parametrize("name", ["unpack_a", "unpack_b"])
def test_oracle_unpack_matches_the_reference_unpack(name):
    """unpack(x, 0) / unpack(x, 1) as the reference's own function computed them (examples/qwen1_5_int8.py:40-50,
    executed by tests/golden/make_golden.py): the oracle's 8-bit accessors give the same bytes."""
    g = np.load(GOLDEN)
    x = g[f"{name}.x"]
    assert np.array_equal(O.unpack_rows(x, 8), g[f"{name}.axis0"])
    assert np.array_equal(O.unpack_cols(x, 8), g[f"{name}.axis1"])
    assert g[f"{name}.axis0"].shape == (x.shape[0] * 4, x.shape[1]) and g[f"{name}.axis1"].shape == (x.shape[0], x.shape[1] * 4)


# ---------------------------------------------------------------------------------------------
# The oracle against the reference's OWN CUDA kernels: tests/golden/ref_cuda_golden.npz holds what those kernels
# (built unchanged from the reference's source strings by oracle/build_ref_cuda.py) produced on a B200
# (tests/golden/make_cuda_golden.py).
# ---------------------------------------------------------------------------------------------
REF_CUDA = os.path.join(os.path.dirname(__file__), "golden", "ref_cuda_golden.npz")


def _h(a):
    return torch.from_numpy(a).view(torch.float16)


def _ulps_fp16(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in representable fp16 values (same sign assumed where it matters)."""
    ia, ib = a.contiguous().view(torch.int16).int(), b.contiguous().view(torch.int16).int()
    return int((ia - ib).abs().max())


@pytest.mark.parametrize("i", range(4))
def test_oracle_matches_the_reference_fused_kernel(i):
    """examples/qwen1_5_int8.py:156-216 run on the GPU: 8-bit, contiguous and act-order groups, 1 to 16 rows.  That kernel
    adds one fp16-rounded partial sum per 32 values of k into the output with atomicAdd (any order), so it agrees with
    the dequantize-then-matmul contract only to the north-star bound, not bit for bit."""
    f = np.load(REF_CUDA)
    x, sc = _h(f[f"qmm{i}_x"]), _h(f[f"qmm{i}_scales"])
    qw, qz, g = (torch.from_numpy(f[f"qmm{i}_{k}"]) for k in ("qweight", "qzeros", "g_idx"))
    ref_kernel = _h(f[f"qmm{i}_out"])
    ours = O.qlinear(x, O.dequantize_packed(qw, g, qz, sc, 8))
    ok, err, bound = O.tolerance_ok(ref_kernel, ours, 1e-2)
    assert ok, f"case {i}: |reference kernel - oracle| = {err} > {bound}"


@pytest.mark.parametrize("i", range(3))
def test_oracle_rms_norm_matches_the_reference_kernel(i):
    """minit/cuda/kernel/cuda/rms_norm.py:56-97 normalises the middle axis of [a, b, c]; the oracle the last one."""
    f = np.load(REF_CUDA)
    x, w, out = _h(f[f"rms{i}_x"]), _h(f[f"rms{i}_w"]), _h(f[f"rms{i}_out"])
    ours = O.rms_norm(x.permute(0, 2, 1).contiguous(), w).permute(0, 2, 1).contiguous()
    assert _ulps_fp16(ours, out) <= 1                            # the order of the fp32 sum of squares differs
    assert (ours.view(torch.int16) != out.view(torch.int16)).float().mean() < 0.01


@pytest.mark.parametrize("i", range(2))
def test_oracle_rope_matches_the_reference_kernel(i):
    """minit/cuda/kernel/cuda/rope.py:57-85 (float instantiation): adjacent pairs rotated by the angle of (position,
    pair index); the difference is the compiler's fused multiply-add."""
    f = np.load(REF_CUDA)
    x, cos, sin, out = (torch.from_numpy(f[f"rope{i}_{k}"]) for k in ("x", "cos", "sin", "out"))
    ours = torch.stack([O.rope(x[b], cos, sin, 0) for b in range(x.shape[0])])
    assert (ours - out).abs().max().item() <= 1e-6


@pytest.mark.parametrize("i", range(3))
def test_softmax_of_the_attention_oracle_matches_the_reference_kernel(i):
    """minit/cuda/kernel/cuda/softmax.py:55-114 over the middle axis, fp32 inside, one rounding to fp16: what
    O.attention computes with torch.softmax on the fp32 copy.  Case 0 has a row with masked (-inf) positions."""
    f = np.load(REF_CUDA)
    x, out = _h(f[f"smx{i}_x"]), _h(f[f"smx{i}_out"])
    ours = torch.softmax(x.float(), dim=1).half()
    assert _ulps_fp16(ours, out) <= 1
    assert (ours.view(torch.int16) != out.view(torch.int16)).float().mean() < 0.01
