"""The integer tensor-core kernel (MT_FLAG_FORCE_MID: 2 < M, packed weights multiplied as unsigned bytes by two-limb
block-fixed-point activations, scale and zero point folded per 128 values of k) against the oracle, through the C ABI."""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MID = 128


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def run(M, c, bits, bias=None, flags=MID, zeros=True):
    from minit_b200 import _lib
    d = to_dev(c, DEV)
    out = M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"] if zeros else None, d["scales"], None,
                                      bits=bits, bias=None if bias is None else bias.to(DEV), flags=flags)
    torch.cuda.synchronize()
    _lib.raise_on_error_words()
    return out


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("bits,dtype", [(4, torch.float16), (4, torch.bfloat16), (8, torch.float16), (8, torch.bfloat16)])
def test_batch_sizes_and_dtypes(M, bits, dtype, m):
    c = O.make_gptq_case(1024, 768, m, bits=bits, dtype=dtype, seed=m)
    assert_close(run(M, c, bits), oracle_out(c, False), f"mid bits={bits} {dtype} M={m}")


@pytest.mark.parametrize("m", [65, 100, 192])
def test_more_than_one_pass(M, m):
    c = O.make_gptq_case(2048, 512, m, bits=4, seed=m)
    assert_close(run(M, c, 4), oracle_out(c, False), f"mid M={m}")


@pytest.mark.parametrize("k,n", [(4096, 4096), (8192, 512), (4096, 14336), (14336, 4096), (128, 32), (256, 96), (2048, 1120)])
@pytest.mark.parametrize("m", [4, 24, 48])
def test_shapes_stream_k_and_ragged_n(M, k, n, m):
    """Deep K (many CTAs per column tile), wide N (runs that cross tiles), N not a multiple of the tile width."""
    c = O.make_gptq_case(k, n, m, bits=4, seed=k + n + m)
    assert_close(run(M, c, 4), oracle_out(c, False), f"mid {k}x{n} M={m}")


@pytest.mark.parametrize("gs", [128, 256, 1024])
@pytest.mark.parametrize("bits", [4, 8])
def test_group_sizes(M, gs, bits):
    c = O.make_gptq_case(2048, 512, 5, bits=bits, group_size=gs, seed=gs)
    assert_close(run(M, c, bits), oracle_out(c, False), f"mid group {gs} bits {bits}")


def test_every_q_and_zero_value(M):
    """All 16 x 16 (q, z) pairs in one column block, so a wrong nibble order or a missing + 1 on the zero shows."""
    c = O.make_gptq_case(256, 256, 7, bits=4, seed=3)
    for z in range(16):
        c["z"][:, z * 16:(z + 1) * 16] = z
    for kk in range(256):
        c["q"][kk, :] = (kk + torch.arange(256).numpy()) % 16
    c["qweight"] = torch.from_numpy(O.pack_rows(c["q"], 4))
    c["qzeros"] = torch.from_numpy(O.pack_cols(c["z"], 4))
    assert_close(run(M, c, 4), oracle_out(c, False), "every (q, z) pair")


def test_rows_of_very_different_magnitude(M):
    """The block scale is per batch row: a row a thousand times smaller than its neighbour keeps its own precision;
    zero rows, huge values and values below the fp16 normal range stay inside the bound."""
    c = O.make_gptq_case(1024, 256, 6, bits=4, seed=21)
    x = c["x"].float()
    x[1] *= 1e-3          # (its outputs stay in the fp16 normal range, so the bound is not below one output ulp)
    x[2] *= 3e3
    x[3] = 0
    x[4, ::2] *= 1e-4
    x[5, 100] = 6e4
    c["x"] = x.half()
    out = run(M, c, 4)
    ref = oracle_out(c, False)
    for r in range(6):
        assert_close(out[r:r + 1], ref[r:r + 1], f"row {r}")


def test_bias_null_zeros_deterministic_and_clean(M):
    from minit_b200 import _lib
    c = O.make_gptq_case(8192, 512, 9, bits=4, seed=77, bias=True)
    a = run(M, c, 4, bias=c["bias"])
    b = run(M, c, 4, bias=c["bias"])
    assert_close(a, oracle_out(c, False, c["bias"]), "mid bias")
    assert torch.equal(a, b)
    ref0 = O.qlinear(c["x"], O.dequantize_packed(c["qweight"], None, None, c["scales"], 4))
    assert_close(run(M, c, 4, zeros=False), ref0, "mid null zeros")
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0    # counters and error word


def test_pdl_back_to_back(M):
    c = O.make_gptq_case(2048, 1024, 12, bits=4, seed=5)
    ref = oracle_out(c, False)
    for _ in range(3):
        out = run(M, c, 4, flags=MID | 4)
    assert_close(out, ref, "mid with programmatic dependent launch")


def test_unsupported_is_refused(M):
    c = O.make_gptq_case(1024, 256, 4, bits=4, group_size=64, seed=1)       # groups of 64: not a multiple of the k-block
    with pytest.raises(RuntimeError):
        run(M, c, 4)


@pytest.mark.parametrize("k,n,ms", [(3072, 2688, (16, 17, 32, 33)),        # 8.3 M weights: the integer kernel from 17 rows on
                                    (4096, 10240, (8, 9, 16, 17)),          # 42 M: from 9 rows on
                                    (2048, 8192, (5, 32)),                  # K < 3072: never
                                    (8192, 14336, (3, 8, 32))])             # 117 M: from 3 rows on
def test_default_dispatch_on_both_sides_of_the_size_rule(M, k, n, ms):
    """mt_qgemm with no flags picks the integer tensor-core kernel or the register-ring kernel by rows and weight size
    (mid_preferred in csrc/api.cu); either way the result is inside the bound.  Checked on a 512-column slice for the
    large weights so that the oracle stays quick."""
    for m in ms:
        c = O.make_gptq_case(k, n, m, bits=4, seed=k // 64 + n // 64 + m)
        out = run(M, c, 4, flags=0)
        sl = slice(n // 2 - 256, n // 2 + 256)
        w = O.dequantize_packed(c["qweight"][:, sl].contiguous(), None, c["qzeros"][:, sl.start // 8:sl.stop // 8].contiguous(),
                                c["scales"][:, sl].contiguous(), 4)
        assert_close(out[:, sl].cpu(), O.qlinear(c["x"], w), f"default dispatch {k}x{n} M={m}")
