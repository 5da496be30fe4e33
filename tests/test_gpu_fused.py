"""Parity of the fused epilogues of a decoder layer's linears with the oracle, through the C ABI:
the gate / up interleave (bit-exact), silu(gate) * up in the epilogue of the fused gate / up linear,
and the residual add in the epilogue of the output linear.

The reference rounds the linear outputs, the sigmoid, silu and the product to the tensor dtype one
after the other (oracle.swiglu); the fused kernels compute the same expression in fp32 and round
once.  The product of two linear outputs is heavy-tailed, so its tolerance is the GEMM bound
(1e-2 * rms of a linear output) propagated through the expression element by element
(assert_swiglu_close), checked against BOTH an fp32 evaluation and the stepwise oracle.
"""
import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VARIANTS = [0, 1 << 24, 2 << 24]          # GEMV schedule: library's choice, split-K, stream-K


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def gate_up_case(k, half, m, bits, dtype, seed, bias=False, gs=128):
    g = O.make_gptq_case(k, half, m, bits=bits, dtype=dtype, seed=seed, bias=bias, group_size=gs)
    u = O.make_gptq_case(k, half, m, bits=bits, dtype=dtype, seed=seed + 1000, bias=bias, group_size=gs)
    u["x"] = g["x"]                      # both projections read the same activations
    return g, u


def interleaved_on_device(M, g, u, bits, zeros=True, bias=False):
    d = lambda t: t.to(DEV)
    return M.interleave_gate_up((d(g["qweight"]), d(g["qzeros"]) if zeros else None, d(g["scales"]), d(g["bias"]) if bias else None),
                                (d(u["qweight"]), d(u["qzeros"]) if zeros else None, d(u["scales"]), d(u["bias"]) if bias else None),
                                bits=bits)


def linear_fp32(c, bits, zeros=True, bias=False):
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"] if zeros else None, c["scales"], bits)
    acc = c["x"].float() @ w.float()
    if bias:
        acc = acc + c["bias"].float()
    return acc


def ulp(v: torch.Tensor, dtype) -> torch.Tensor:
    """spacing of `dtype` at |v| (normal range)"""
    bits = 10 if dtype == torch.float16 else 7
    return torch.exp2(torch.floor(torch.log2(v.abs().clamp_min(1e-30))) - bits)


def assert_swiglu_close(out, g, u, bits, zeros=True, bias=False, what=""):
    """out against silu(yg) * yu with yg, yu the fp32 linear outputs, and against the stepwise oracle.

    The north-star bound on a linear output y is eps = 1e-2 * rms(y) (plus one ulp of the largest |y| when y is
    rounded to the tensor dtype on the way); through d/dg silu(g) u = silu'(g) u (|silu'| <= 1.1) and
    d/du = silu(g) it becomes eps * (1.1 |yu| + |silu(yg)|) per element of the product, plus the roundings of
    the result itself: one for the fused kernels, three for the reference's separate kernels."""
    T = g["x"].dtype
    yg, yu = linear_fp32(g, bits, zeros, bias), linear_fp32(u, bits, zeros, bias)
    sg = torch.nn.functional.silu(yg)
    exact = sg * yu
    eps = 1e-2 * max(yg.pow(2).mean().sqrt().item(), yu.pow(2).mean().sqrt().item()) + ulp(torch.maximum(yg.abs().max(), yu.abs().max()), T).item()
    prop = eps * (1.1 * yu.abs() + sg.abs())
    o = out.float().cpu()
    bad = (o - exact).abs() > prop + ulp(exact, T) + 1e-6
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond the propagated bound, worst {(o - exact).abs().max().item():.4g}"
    step = O.swiglu(yg.to(T), yu.to(T)).float()
    bad = (o - step).abs() > prop + 3 * ulp(step, T) + 1e-6
    assert not bad.any(), f"{what} (stepwise oracle): {int(bad.sum())} elements beyond the bound, worst {(o - step).abs().max().item():.4g}"
    # and the product is not simply zero / garbage: the usual global bound at 10x
    ok, err, bound = O.tolerance_ok(out, exact.to(T), 1e-1)
    bound += 2 * ulp(exact.abs().max(), T).item()
    assert err <= bound, f"{what}: max abs err {err:.4g} > {bound:.4g}"


def swiglu_refs(g, u, bits, zeros=True, bias=False):
    """(stepwise oracle in T, fp32 evaluation rounded once)"""
    yg, yu = linear_fp32(g, bits, zeros, bias), linear_fp32(u, bits, zeros, bias)
    T = g["x"].dtype
    stepwise = O.swiglu(yg.to(T), yu.to(T))
    exact = (torch.nn.functional.silu(yg) * yu).to(T)
    return stepwise, exact


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("zeros,bias", [(True, True), (True, False), (False, False)])
def test_interleave_is_bit_exact(M, bits, dtype, zeros, bias):
    g, u = gate_up_case(512, 264, 1, bits, dtype, seed=bits + 7, bias=bias)      # 264 = 8 * 33: odd number of column blocks
    qw, qz, sc, bi = interleaved_on_device(M, g, u, bits, zeros, bias)
    rq, rz, rs = O.interleave_gate_up((g["qweight"], g["qzeros"], g["scales"].view(torch.int16)),
                                      (u["qweight"], u["qzeros"], u["scales"].view(torch.int16)), bits)
    assert np.array_equal(qw.cpu().numpy(), rq)
    assert np.array_equal(sc.view(torch.int16).cpu().numpy().view(np.uint16), rs.view(np.uint16))
    if zeros:
        assert np.array_equal(qz.cpu().numpy(), rz)
    else:
        assert qz is None
    if bias:
        rb = O.interleave_columns(g["bias"].view(torch.int16).numpy()[None], u["bias"].view(torch.int16).numpy()[None])[0]
        assert np.array_equal(bi.view(torch.int16).cpu().numpy(), rb)
    # the fused linear on the interleaved layout is the column-interleave of the two linears (same kernel, same bits)
    x = g["x"].to(DEV)
    y = M.quantized_matrix_multiply(x, qw, qz, sc, None, bits=bits, bias=bi)
    d = lambda t: t.to(DEV)
    yg = M.quantized_matrix_multiply(x, d(g["qweight"]), d(g["qzeros"]) if zeros else None, d(g["scales"]), None, bits=bits,
                                     bias=d(g["bias"]) if bias else None)
    yu = M.quantized_matrix_multiply(x, d(u["qweight"]), d(u["qzeros"]) if zeros else None, d(u["scales"]), None, bits=bits,
                                     bias=d(u["bias"]) if bias else None)
    ref = O.interleave_columns(yg.view(torch.int16).cpu().numpy(), yu.view(torch.int16).cpu().numpy())
    assert_close(y.cpu(), torch.from_numpy(ref).view(dtype), "interleaved linear")


@pytest.mark.parametrize("variant", VARIANTS, ids=["auto", "split", "stream"])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("k,half", [(1024, 384), (4096, 1024), (512, 64)])
def test_swiglu_gemv(M, variant, bits, dtype, m, k, half):
    g, u = gate_up_case(k, half, m, bits, dtype, seed=k + half + m)
    qw, qz, sc, _ = interleaved_on_device(M, g, u, bits)
    out = M.quantized_gate_up_swiglu(g["x"].to(DEV), qw, qz, sc, bits=bits, flags=variant)
    assert out.shape == (m, half)
    assert_swiglu_close(out, g, u, bits, what=f"swiglu bits={bits} {dtype} M={m} {k}x{half}")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 2])
def test_swiglu_gemv_bias_and_symmetric(M, bits, m):
    g, u = gate_up_case(2048, 512, m, bits, torch.float16, seed=31 + m, bias=True)
    qw, qz, sc, bi = interleaved_on_device(M, g, u, bits, zeros=True, bias=True)
    out = M.quantized_gate_up_swiglu(g["x"].to(DEV), qw, qz, sc, bits=bits, bias=bi)
    assert_swiglu_close(out, g, u, bits, True, True, "swiglu with bias")
    qw, qz, sc, _ = interleaved_on_device(M, g, u, bits, zeros=False)
    out = M.quantized_gate_up_swiglu(g["x"].to(DEV), qw, None, sc, bits=bits)
    assert_swiglu_close(out, g, u, bits, False, False, "swiglu symmetric zero point")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [3, 16, 48, 100, 300])
def test_swiglu_larger_batches(M, bits, dtype, m):
    """M > 2: GEMM into a scratch tensor, then the stand-alone activation kernel."""
    if bits == 8 and dtype == torch.bfloat16 and m > 64:
        pytest.skip("the prefill kernel has no 8-bit bf16 instantiation")
    g, u = gate_up_case(1024, 256, m, bits, dtype, seed=m)
    qw, qz, sc, _ = interleaved_on_device(M, g, u, bits)
    out = M.quantized_gate_up_swiglu(g["x"].to(DEV), qw, qz, sc, bits=bits)
    assert_swiglu_close(out, g, u, bits, what=f"swiglu M={m}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_swiglu_elementwise_matches_oracle(M, dtype):
    gen = torch.Generator().manual_seed(5)
    yg = (torch.randn((7, 264), generator=gen) * 3).to(dtype)
    yu = (torch.randn((7, 264), generator=gen) * 2).to(dtype)
    y = torch.from_numpy(O.interleave_columns(yg.view(torch.int16).numpy(), yu.view(torch.int16).numpy())).view(dtype)
    out = M.swiglu_interleaved(y.to(DEV)).cpu()
    exact = (torch.nn.functional.silu(yg.float()) * yu.float())
    # one rounding of the fp32 value: half an ulp
    ulp = 2.0 ** (-11 if dtype == torch.float16 else -8)
    assert ((out.float() - exact).abs() <= exact.abs() * ulp * 1.01 + 1e-7).all()
    # the stepwise oracle rounds three times: within 2.5 ulp of it
    step = O.swiglu(yg, yu).float()
    assert ((out.float() - step).abs() <= step.abs() * ulp * 5 + 1e-6).all()


@pytest.mark.parametrize("variant", VARIANTS, ids=["auto", "split", "stream"])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2])
def test_residual_gemv(M, variant, bits, dtype, m):
    c = O.make_gptq_case(2048, 1024, m, bits=bits, dtype=dtype, seed=11 + m, bias=True)
    gen = torch.Generator().manual_seed(3)
    res = (torch.randn((m, 1024), generator=gen) * 2).to(dtype)
    d = lambda t: t.to(DEV)
    out = M.quantized_matrix_multiply_residual(d(c["x"]), d(c["qweight"]), d(c["qzeros"]), d(c["scales"]), None, d(res),
                                               bits=bits, bias=d(c["bias"]), flags=variant)
    y32 = linear_fp32(c, bits, True, True)
    assert_close(out, (y32 + res.float()).to(dtype), "residual vs fp32")
    assert_close(out, O.add_residual(res, y32.to(dtype)), "residual vs stepwise oracle")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [5, 40, 200])
@pytest.mark.parametrize("act_order", [False, True])
def test_residual_larger_batches_match_the_reference_steps(M, bits, m, act_order):
    """M > 2 (and act-order at any M): GEMM, then one elementwise add -- the reference's two roundings, so the
    result equals add_residual(residual, linear output) bit for bit given the linear output."""
    c = O.make_gptq_case(1024, 512, m, bits=bits, seed=m, act_order=act_order)
    gen = torch.Generator().manual_seed(4)
    res = torch.randn((m, 512), generator=gen).half()
    d = lambda t: t.to(DEV)
    groups = d(c["g_idx"]) if act_order else None
    y = M.quantized_matrix_multiply(d(c["x"]), d(c["qweight"]), d(c["qzeros"]), d(c["scales"]), groups, bits=bits)
    out = M.quantized_matrix_multiply_residual(d(c["x"]), d(c["qweight"]), d(c["qzeros"]), d(c["scales"]), groups, d(res), bits=bits)
    assert torch.equal(out.cpu(), O.add_residual(res, y.cpu()))


@pytest.mark.parametrize("m", [1, 2, 24])
@pytest.mark.parametrize("names,bias", [(("gate_proj", "up_proj", "down_proj"), False), (("w2", "w1", "c_proj"), True)])
def test_feed_forward_module(M, m, names, bias):
    """QFeedForward against the reference composition down(silu(gate(x)) * up(x)) (+ residual) from the oracle."""
    hidden, inner, bits = 512, 1024, 4
    g, u = gate_up_case(hidden, inner, m, bits, torch.float16, seed=77, bias=bias)
    dn = O.make_gptq_case(inner, hidden, m, bits=bits, seed=78, bias=bias)
    ff = M.QFeedForward(hidden, inner, hidden // 128, inner // 128, bits=bits, bias=bias, names=names)
    for name, c in zip(names, (g, u, dn)):
        for buf in ("qweight", "qzeros", "scales", "g_idx") + (("bias",) if bias else ()):
            ff.update_buffer(f"{name}.{buf}", c[buf].to(DEV))
    x = g["x"]
    res = torch.randn((m, hidden), generator=torch.Generator().manual_seed(9)).half()
    h_ref = swiglu_refs(g, u, bits, True, bias)[0]
    wd = O.dequantize_packed(dn["qweight"], None, dn["qzeros"], dn["scales"], bits)
    y_ref = O.qlinear(h_ref, wd, dn["bias"] if bias else None)
    assert_close(ff(x.to(DEV)), y_ref, "feed-forward")
    assert_close(ff(x.to(DEV), residual=res.to(DEV)), O.add_residual(res, y_ref), "feed-forward + residual")


@pytest.mark.parametrize("m", [1, 2])
def test_shapes_the_gemv_does_not_take_fall_back(M, m):
    """N not a multiple of 128 (the GEMV's column block): the two-launch path serves M <= 2 as well; empty batches are a no-op."""
    bits = 4
    g, u = gate_up_case(512, 200, m, bits, torch.float16, seed=3)                   # N = 400
    qw, qz, sc, _ = interleaved_on_device(M, g, u, bits)
    out = M.quantized_gate_up_swiglu(g["x"].to(DEV), qw, qz, sc, bits=bits)
    assert_swiglu_close(out, g, u, bits, what="swiglu N=400")
    c = O.make_gptq_case(512, 200, m, bits=bits, seed=5)
    res = torch.randn((m, 200), generator=torch.Generator().manual_seed(1)).half()
    d = lambda t: t.to(DEV)
    out = M.quantized_matrix_multiply_residual(d(c["x"]), d(c["qweight"]), d(c["qzeros"]), d(c["scales"]), None, d(res), bits=bits)
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], bits)
    assert_close(out, O.add_residual(res, O.qlinear(c["x"], w)), "residual N=200")
    empty = M.quantized_gate_up_swiglu(g["x"][:0].to(DEV), qw, qz, sc, bits=bits)
    assert empty.shape == (0, 200)
    empty = M.quantized_matrix_multiply_residual(d(c["x"][:0]), d(c["qweight"]), d(c["qzeros"]), d(c["scales"]), None, d(res[:0]), bits=bits)
    assert empty.shape == (0, 200)


def test_status_codes(M):
    from minit_b200 import _lib
    lib = _lib.lib
    z = torch.zeros(4096, dtype=torch.int32, device=DEV)
    p = z.data_ptr()
    assert lib.mt_qgemm_swiglu(None, p, p, p, p, None, p, None, 1, 24, 256, 2, 4, 0, None, 0, 0) == -3       # N % 16
    assert lib.mt_qgemm_swiglu(None, p, p, p, p, None, p, None, 8, 32, 256, 2, 4, 0, p, 16384, 0) == -1      # scratch missing at M > 2
    assert lib.mt_interleave_gate_up(None, p, p, p, None, p, p, None, None, p, p, p, None, 64, 256, 2, 4) == -1   # zeros of one side only
    assert lib.mt_interleave_gate_up(None, p, p, None, None, p, p, None, None, p, None, p, None, 12, 256, 2, 4) == -3
    assert lib.mt_swiglu(None, p, p, 1, 24, 0) == -3
    assert lib.mt_swiglu(None, p, p, 1, 32, 7) == -4


def test_full_size_feed_forward_block(M):
    """Llama-3-70B feed-forward at full size (8192 -> 2 x 28672 -> 8192), M = 1: the fused two-kernel form against the
    separate launches of the same library (same weights), and a column slice of the first stage against the oracle."""
    hidden, inner, bits = 8192, 28672, 4
    gen = torch.Generator(device=DEV).manual_seed(0)

    def rnd(k, n):
        qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), device=DEV, dtype=torch.int64, generator=gen).to(torch.int32)
        qz = torch.randint(-2**31, 2**31 - 1, (k // 128, n // 8), device=DEV, dtype=torch.int64, generator=gen).to(torch.int32)
        sc = (0.0005 + 0.001 * torch.rand((k // 128, n), device=DEV, generator=gen)).half()
        return qw, qz, sc
    gq, gz, gs = rnd(hidden, inner)
    uq, uz, us = rnd(hidden, inner)
    dq, dz, ds = rnd(inner, hidden)
    x = torch.randn((1, hidden), device=DEV, generator=gen).half()
    res = torch.randn((1, hidden), device=DEV, generator=gen).half()
    qw, qz, sc, _ = M.interleave_gate_up((gq, gz, gs, None), (uq, uz, us, None), bits=bits)
    h = M.quantized_gate_up_swiglu(x, qw, qz, sc, bits=bits)
    out = M.quantized_matrix_multiply_residual(h, dq, dz, ds, None, res, bits=bits)
    # the same block as four launches
    yg = M.quantized_matrix_multiply(x, gq, gz, gs, None, bits=bits)
    yu = M.quantized_matrix_multiply(x, uq, uz, us, None, bits=bits)
    h2 = (torch.nn.functional.silu(yg.float()) * yu.float()).half()
    assert_close(h, h2, "fused activation vs separate linears")
    out2 = (M.quantized_matrix_multiply(h2, dq, dz, ds, None, bits=bits).float() + res.float()).half()
    assert_close(out, out2, "fused block vs separate launches")
    # oracle on gate / up columns 20000 .. 20063
    lo, hi = 20000, 20064
    cpu = lambda t: t.cpu()
    wg = O.dequantize_packed(cpu(gq[:, lo:hi]).contiguous(), None, cpu(gz[:, lo // 8:hi // 8]).contiguous(), cpu(gs[:, lo:hi]).contiguous(), bits)
    wu = O.dequantize_packed(cpu(uq[:, lo:hi]).contiguous(), None, cpu(uz[:, lo // 8:hi // 8]).contiguous(), cpu(us[:, lo:hi]).contiguous(), bits)
    ref = O.swiglu(O.qlinear(cpu(x), wg), O.qlinear(cpu(x), wu))
    assert_close(h[:, lo:hi].cpu(), ref, "fused activation vs oracle slice")
