"""The mid-batch tcgen05 kernel (MT_FLAG_FORCE_UMMA: 2 < M <= 192, all warps dequantize, weights reach the
tensor core through tensor memory) against the oracle, through the C ABI."""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
UMMA = 32


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def run(M, c, bits, bias=None, flags=UMMA, zeros=True):
    d = to_dev(c, DEV)
    return M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"] if zeros else None, d["scales"], None,
                                       bits=bits, bias=None if bias is None else bias.to(DEV), flags=flags)


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("bits,dtype", [(4, torch.float16), (4, torch.bfloat16), (8, torch.float16)])
def test_batch_sizes_and_dtypes(M, bits, dtype, m):
    c = O.make_gptq_case(1024, 768, m, bits=bits, dtype=dtype, seed=m)
    assert_close(run(M, c, bits), oracle_out(c, False), f"umma bits={bits} {dtype} M={m}")


@pytest.mark.parametrize("m", [65, 100, 192])
def test_more_than_one_pass(M, m):
    c = O.make_gptq_case(2048, 512, m, bits=4, seed=m)
    assert_close(run(M, c, 4), oracle_out(c, False), f"umma M={m}")


@pytest.mark.parametrize("k,n", [(4096, 4096), (8192, 512), (4096, 14336), (14336, 4096), (64, 256), (128, 8), (2048, 1000)])
@pytest.mark.parametrize("m", [4, 48])
def test_shapes_stream_k_and_ragged_n(M, k, n, m):
    """Deep K (many CTAs per column tile), wide N (runs that cross tiles), N not a multiple of 256."""
    gs = 64 if k < 128 else 128
    c = O.make_gptq_case(k, n, m, bits=4, group_size=gs, seed=k + n + m)
    assert_close(run(M, c, 4), oracle_out(c, False), f"umma {k}x{n} M={m}")


@pytest.mark.parametrize("gs", [64, 128, 256, 1024])
@pytest.mark.parametrize("bits", [4, 8])
def test_group_sizes(M, gs, bits):
    c = O.make_gptq_case(2048, 512, 5, bits=bits, group_size=gs, seed=gs)
    assert_close(run(M, c, bits), oracle_out(c, False), f"umma group {gs} bits {bits}")


def test_bias_null_zeros_deterministic_and_clean(M):
    from minit_b200 import _lib
    c = O.make_gptq_case(8192, 512, 9, bits=4, seed=77, bias=True)
    a = run(M, c, 4, bias=c["bias"])
    b = run(M, c, 4, bias=c["bias"])
    assert_close(a, oracle_out(c, False, c["bias"]), "umma bias")
    assert torch.equal(a, b)
    ref0 = O.qlinear(c["x"], O.dequantize_packed(c["qweight"], None, None, c["scales"], 4))
    assert_close(run(M, c, 4, zeros=False), ref0, "umma null zeros")
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0    # counters and error word


def test_unsupported_is_refused(M):
    c = O.make_gptq_case(1024, 256, 4, bits=4, group_size=32, seed=1)       # groups of 32: not a multiple of the k-block
    with pytest.raises(RuntimeError):
        run(M, c, 4)
    c = O.make_gptq_case(1024, 256, 4, bits=8, dtype=torch.bfloat16, seed=1)
    with pytest.raises(RuntimeError):
        run(M, c, 8)
