"""mt_qgemm decode kernels through the C ABI against the oracle: flags=1 forces the register-ring
kernel (mma.sync), flags=0 lets the library choose.
Tolerance from the north star: max|out - ref| <= 1e-2 * rms(ref), ref = T(float(x) @ float(W_oracle))."""
import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def run(M, c, act, bits, bias=None, flags=1):
    d = to_dev(c, DEV)
    return M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"], d["scales"], d["g_idx"] if act else None,
                                       bits=bits, bias=None if bias is None else bias.to(DEV), flags=flags)


KERNELS = [0, 1]


@pytest.mark.parametrize("flags", KERNELS)
@pytest.mark.parametrize("m", [1, 16])
def test_config1_single_int4_linear(M, m, flags):
    c = O.make_gptq_case(4096, 4096, m, bits=4, seed=0)
    assert_close(run(M, c, False, 4, flags=flags), oracle_out(c, False), f"cfg1 M={m}")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("flags", KERNELS)
def test_batch_sizes_and_dtypes(M, bits, dtype, m, flags):
    if flags == 8 and (m > 16 or (bits == 8 and dtype == torch.bfloat16)):
        pytest.skip("outside the tcgen05 decode kernel's range")
    c = O.make_gptq_case(1024, 768, m, bits=bits, dtype=dtype, seed=m)
    assert_close(run(M, c, False, bits, flags=flags), oracle_out(c, False), f"bits={bits} {dtype} M={m}")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_act_order(M, bits, dtype, m):
    c = O.make_gptq_case(1024, 512, m, bits=bits, act_order=True, dtype=dtype, seed=20 + m)
    assert_close(run(M, c, True, bits), oracle_out(c, True), f"act-order bits={bits} {dtype} M={m}")


@pytest.mark.parametrize("k,n", [(4096, 1024), (4096, 14336), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 64])
def test_config3_mistral_shapes_act_order(M, k, n, m):
    c = O.make_gptq_case(k, n, m, bits=4, act_order=True, seed=k + n + m)
    assert_close(run(M, c, True, 4), oracle_out(c, True), f"cfg3 {k}x{n} M={m}")


@pytest.mark.parametrize("gs", [32, 64, 128, 256, 1024])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("flags", KERNELS)
def test_group_sizes(M, gs, bits, flags):
    if flags == 8 and gs < 64:
        pytest.skip("the tcgen05 decode kernel folds in units of 64 k")
    c = O.make_gptq_case(1024, 256, 5, bits=bits, group_size=gs, seed=gs)
    assert_close(run(M, c, False, bits, flags=flags), oracle_out(c, False), f"group {gs} bits {bits}")


@pytest.mark.parametrize("k,n", [(32, 8), (96, 40), (1056, 8), (2080, 1000), (11008, 264)])
@pytest.mark.parametrize("flags", KERNELS)
def test_ragged_shapes(M, k, n, flags):
    """K not a multiple of the 256-wide chunk, N not a multiple of the column tile."""
    gs = 32 if k % 128 else 128
    if flags == 8 and gs < 64:
        pytest.skip("the tcgen05 decode kernel folds in units of 64 k")
    c = O.make_gptq_case(k, n, 7, bits=4, group_size=gs, seed=k)
    assert_close(run(M, c, False, 4, flags=flags), oracle_out(c, False), f"ragged {k}x{n}")
    c8 = O.make_gptq_case(k, n, 2, bits=8, group_size=gs, seed=k + 1)
    assert_close(run(M, c8, False, 8, flags=flags), oracle_out(c8, False), f"ragged int8 {k}x{n}")


@pytest.mark.parametrize("flags", KERNELS)
def test_bias_null_zeros_and_output_is_overwritten(M, flags):
    c = O.make_gptq_case(512, 256, 4, bits=4, seed=77, bias=True)
    out = run(M, c, False, 4, bias=c["bias"], flags=flags)
    assert_close(out, oracle_out(c, False, c["bias"]), "bias")
    d = to_dev(c, DEV)
    ref0 = O.qlinear(c["x"], O.dequantize_packed(c["qweight"], None, None, c["scales"], 4))
    buf = torch.full((4, 256), 1000.0, dtype=torch.float16, device=DEV)   # garbage that must not be accumulated into
    M.quantized_matrix_multiply(d["x"], d["qweight"], None, d["scales"], None, bits=4, out=buf, flags=flags)
    assert_close(buf, ref0, "null zeros / overwrite")


def test_leading_dims_fold_and_empty_batch(M):
    c = O.make_gptq_case(256, 64, 6, bits=4, seed=5)
    d = to_dev(c, DEV)
    x3 = d["x"].reshape(2, 3, 256)
    out = M.quantized_matrix_multiply(x3, d["qweight"], d["qzeros"], d["scales"], None, bits=4)
    assert out.shape == (2, 3, 64)
    assert_close(out.reshape(6, 64), oracle_out(c, False), "folded dims")
    empty = M.quantized_matrix_multiply(d["x"][:0], d["qweight"], d["qzeros"], d["scales"], None, bits=4)
    assert empty.shape == (0, 64)


def test_m_above_64_tiles_through_the_small_kernel(M):
    c = O.make_gptq_case(512, 256, 150, bits=4, seed=8)
    assert_close(run(M, c, False, 4, flags=1), oracle_out(c, False), "M=150 forced small")


@pytest.mark.parametrize("flags", KERNELS)
def test_deterministic_and_workspace_left_clean(M, flags):
    from minit_b200 import _lib
    c = O.make_gptq_case(8192, 512, 2, bits=4, seed=4)    # deep K -> split-K is active
    a = run(M, c, False, 4, flags=flags)
    b = run(M, c, False, 4, flags=flags)
    assert torch.equal(a, b)
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


@pytest.mark.parametrize("flags", KERNELS)
def test_pdl_launch_flag(M, flags):
    c = O.make_gptq_case(2048, 512, 1, bits=4, seed=12)
    ref = oracle_out(c, False)
    for _ in range(3):
        out = run(M, c, False, 4, flags=flags | 4)
    assert_close(out, ref, "PDL launches back to back")


def test_large_scales_and_small_x_stay_inside_tolerance(M):
    """Scales up to 1 and x values that underflow when divided by 16 must not break the bound."""
    c = O.make_gptq_case(4096, 256, 3, bits=4, seed=31, scale_lo=0.5, scale_hi=1.0)
    assert_close(run(M, c, False, 4, flags=0), oracle_out(c, False), "large scales")
    c = O.make_gptq_case(4096, 256, 3, bits=4, seed=32)
    c["x"] = (c["x"].float() * 1e-4).half()
    assert_close(run(M, c, False, 4, flags=0), oracle_out(c, False), "tiny x")


def test_full_size_linearity_property(M):
    """Largest decode shape of the 70B config on one GPU (8192 -> 57344, M=1): checked through
    linearity, out(x1 + x2) ~= out(x1) + out(x2), and against the oracle on a column slice."""
    k, n = 8192, 57344
    gen = torch.Generator().manual_seed(1)
    qw = torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=gen, dtype=torch.int64).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (k // 128, n // 8), generator=gen, dtype=torch.int64).to(torch.int32)
    s = (0.002 + 0.018 * torch.rand((k // 128, n), generator=gen)).half()
    x1 = torch.randn((1, k), generator=gen).half()
    x2 = torch.randn((1, k), generator=gen).half()
    f = lambda x: M.quantized_matrix_multiply(x.to(DEV), qw.to(DEV), qz.to(DEV), s.to(DEV), None, bits=4).float().cpu()
    o1, o2, o12 = f(x1), f(x2), f((x1.float() + x2.float()).half())
    rms = o12.pow(2).mean().sqrt()
    assert (o12 - (o1 + o2)).abs().max() <= 2e-2 * rms
    sl = slice(4096, 4096 + 512)
    w = O.dequantize_packed(qw[:, sl].contiguous(), None, qz[:, 512:576].contiguous(), s[:, sl].contiguous(), 4)
    assert_close(o1[:, sl], O.qlinear(x1, w), "column slice of the full-size linear")


@pytest.mark.parametrize("m,k,n,bits", [(2, 8192, 57344, 4), (32, 8192, 57344, 4), (64, 28672, 8192, 4), (1, 8192, 28672, 8)])
def test_full_size_shapes_every_dispatch_path(M, m, k, n, bits):
    """The 70B linears at the batch sizes each decode kernel serves (GEMV stream-K, mid-batch tcgen05 kernel, 8-bit GEMV):
    linearity in x, and the oracle on a slice of columns that starts inside a column tile."""
    pack = 32 // bits
    gen = torch.Generator().manual_seed(m + k)
    qw = torch.randint(-2**31, 2**31 - 1, (k // pack, n), generator=gen, dtype=torch.int64).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (k // 128, n // pack), generator=gen, dtype=torch.int64).to(torch.int32)
    s = (0.002 + 0.018 * torch.rand((k // 128, n), generator=gen)).half()
    x1 = torch.randn((m, k), generator=gen).half()
    x2 = torch.randn((m, k), generator=gen).half()
    dq, dz, ds = qw.to(DEV), qz.to(DEV), s.to(DEV)
    f = lambda x: M.quantized_matrix_multiply(x.to(DEV), dq, dz, ds, None, bits=bits).float().cpu()
    o1, o2, o12 = f(x1), f(x2), f((x1.float() + x2.float()).half())
    rms = o12.pow(2).mean().sqrt()
    assert (o12 - (o1 + o2)).abs().max() <= 2e-2 * rms
    c0 = 4096 + 64                                           # not a multiple of 128 or 256
    sl = slice(c0, c0 + 512)
    w = O.dequantize_packed(qw[:, sl].contiguous(), None, qz[:, c0 // pack:(c0 + 512) // pack].contiguous(), s[:, sl].contiguous(), bits)
    assert_close(o1[:, sl], O.qlinear(x1, w), f"column slice of {k}x{n} M={m} bits={bits}")
