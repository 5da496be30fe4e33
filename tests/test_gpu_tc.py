"""The tcgen05 prefill kernel (forced with MT_FLAG_FORCE_TC) through the C ABI against the oracle."""
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


def run(M, c, bits, bias=None, flags=2):
    from minit_b200 import _lib
    d = to_dev(c, DEV)
    out = M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"], d["scales"], None, bits=bits,
                                      bias=None if bias is None else bias.to(DEV), flags=flags)
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert _lib.workspace_error_word(ws) == 0, "a bounded wait inside the tcgen05 kernel expired"
    return out


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [64, 128, 256, 300, 1000])
def test_tc_matches_oracle(M, bits, dtype, m):
    c = O.make_gptq_case(1024, 512, m, bits=bits, dtype=dtype, seed=m)
    assert_close(run(M, c, bits), oracle_out(c, False), f"tc bits={bits} {dtype} M={m}")


@pytest.mark.parametrize("k,n", [(64, 128), (192, 136), (4096, 6144), (2048, 1000)])
def test_tc_shapes_edges_bias(M, k, n):
    c = O.make_gptq_case(k, n, 260, bits=4, group_size=64, seed=k + n, bias=True)
    assert_close(run(M, c, 4, bias=c["bias"]), oracle_out(c, False, c["bias"]), f"tc {k}x{n}")


def test_tc_many_tiles_per_cta_and_both_accumulators(M):
    """More tiles than SMs so every persistent CTA loops and alternates its two TMEM accumulators."""
    c = O.make_gptq_case(512, 128 * 40, 2048, bits=4, seed=9)
    assert_close(run(M, c, 4), oracle_out(c, False), "tc 320 tiles")


def test_tc_is_the_default_above_64_rows(M):
    c = O.make_gptq_case(1024, 256, 200, bits=4, seed=2)
    assert_close(run(M, c, 4, flags=0), oracle_out(c, False), "default dispatch M=200")


def test_tc_prefill_shape_4096(M):
    """Prefill config: (K,N) = (4096, 6144), M = 4096, bf16; oracle on 3 row blocks to bound CPU time."""
    c = O.make_gptq_case(4096, 6144, 4096, bits=4, dtype=torch.bfloat16, seed=1)
    out = run(M, c, 4).cpu()
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4)
    for r0 in (0, 2000, 3968):
        assert_close(out[r0:r0 + 128], O.qlinear(c["x"][r0:r0 + 128], w), f"prefill rows {r0}")


# The prefill config's other shapes at every batch size it names, in both dtypes.  One case per
# (shape, dtype) is built at the largest M and its leading rows serve the smaller ones; the oracle
# checks three 128-row blocks of each output to bound CPU time.
_PREFILL_CASES = {}


def _prefill_case(k, n, dtype):
    key = (k, n, dtype)
    if key not in _PREFILL_CASES:
        _PREFILL_CASES.clear()                      # one resident case at a time (hundreds of MB each)
        c = O.make_gptq_case(k, n, 8192, bits=4, dtype=dtype, seed=k + n)
        c.pop("q"); c.pop("z")
        c["w"] = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4)
        _PREFILL_CASES[key] = c
    return _PREFILL_CASES[key]


@pytest.mark.parametrize("m", [2048, 4096, 8192])       # the top decorator varies fastest: a case is built once
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k,n", [(4096, 28672), (14336, 4096)])
def test_tc_prefill_config_shapes(M, k, n, dtype, m):
    c = _prefill_case(k, n, dtype)
    d = {key: val for key, val in c.items() if key != "w"}
    d["x"] = c["x"][:m].contiguous()
    out = run(M, d, 4, flags=0).cpu()                 # default dispatch: what a caller of this config gets
    assert tuple(out.shape) == (m, n)
    for r0 in (0, m // 2 - 64, m - 128):
        assert_close(out[r0:r0 + 128], O.qlinear(d["x"][r0:r0 + 128], c["w"]), f"prefill {k}x{n} M={m} {dtype} rows {r0}")


TMEM_A = 2 | 256          # MT_FLAG_FORCE_TC | MT_FLAG_TC_TMEM_A: the 256 x 192 tile with the dequantized weights in tensor memory


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [129, 192, 193, 256, 400, 1000])
def test_tensor_memory_operand_variant_matches_oracle(M, dtype, m):
    """Row counts on both sides of the 192-row tile; K = 1024 gives 16 k-blocks, so both converter groups and both
    slots of A in tensor memory are reused."""
    c = O.make_gptq_case(1024, 512, m, bits=4, dtype=dtype, seed=m + 1)
    assert_close(run(M, c, 4, flags=TMEM_A), oracle_out(c, False), f"tensor-memory A {dtype} M={m}")


@pytest.mark.parametrize("k,n", [(64, 256), (192, 264), (4096, 6144), (2048, 1000), (448, 512)])
def test_tensor_memory_operand_variant_shapes_edges_bias(M, k, n):
    """One k-block, an odd number of k-blocks (the groups swap slots from tile to tile), ragged N, bias."""
    c = O.make_gptq_case(k, n, 260, bits=4, group_size=64, seed=k + n + 1, bias=True)
    assert_close(run(M, c, 4, bias=c["bias"], flags=TMEM_A), oracle_out(c, False, c["bias"]), f"tensor-memory A {k}x{n}")


def test_tensor_memory_operand_variant_many_tiles_per_cta(M):
    c = O.make_gptq_case(512, 256 * 24, 2048, bits=4, seed=10)
    assert_close(run(M, c, 4, flags=TMEM_A), oracle_out(c, False), "tensor-memory A, 264 tiles")


@pytest.mark.parametrize("k,n,m,dtype,bias", [(2048, 4096, 1920, torch.float16, False),     # 160 tiles: the last 12 are cut in 2 along K
                                              (4096, 4096, 1900, torch.bfloat16, True),     # cut in 4, ragged last row tile, bias
                                              (1024, 4352, 1728, torch.float16, False)])    # 153 tiles, 16 k-blocks: too short to cut
def test_last_wave_of_tiles_cut_along_k(M, k, n, m, dtype, bias):
    """More tiles than SMs with a small remainder: the remaining tiles are split along K, their fp32 partial tiles are
    added in part order by whichever part arrives last, and the workspace counters return to zero."""
    from minit_b200 import _lib
    c = O.make_gptq_case(k, n, m, bits=4, dtype=dtype, seed=k + n + m, bias=bias)
    b = c["bias"] if bias else None
    out1 = run(M, c, 4, bias=b, flags=TMEM_A)
    out2 = run(M, c, 4, bias=b, flags=TMEM_A)
    assert torch.equal(out1, out2), "the split tiles must not depend on which part arrives last"
    assert_close(out1, oracle_out(c, False, b), f"split last wave {k}x{n} M={m}")
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


@pytest.mark.parametrize("k,n", [(2048, 512), (8192, 1024), (1024, 4352), (512, 264)])
@pytest.mark.parametrize("m,dtype", [(3, torch.float16), (33, torch.float16), (64, torch.bfloat16)])
def test_tensor_memory_operand_variant_with_64_row_tiles(M, k, n, m, dtype):
    """Up to 64 rows the same kernel runs with 64-row tiles, every tile cut along K into parts that are added in part
    order (deep K: up to 8 parts; K = 512: no cut); results repeat bit for bit and the counters return to zero."""
    from minit_b200 import _lib
    c = O.make_gptq_case(k, n, m, bits=4, dtype=dtype, seed=k + n + m + 5, bias=True)
    out1 = run(M, c, 4, bias=c["bias"], flags=TMEM_A)
    out2 = run(M, c, 4, bias=c["bias"], flags=TMEM_A)
    assert torch.equal(out1, out2)
    assert_close(out1, oracle_out(c, False, c["bias"]), f"64-row tiles {k}x{n} M={m}")
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


@pytest.mark.parametrize("k,n", [(2048, 1024), (8192, 512), (1024, 4352)])
@pytest.mark.parametrize("m", [33, 64, 65, 100, 160, 161, 192])
def test_default_dispatch_33_to_192_rows(M, k, n, m):
    """mt_qgemm with no flags: 33 to 192 rows on int4 weights with contiguous groups go to one row of tiles (64, 160 or 192
    rows) of the tensor-memory-A kernel, every tile cut along K where that fills the GPU better."""
    c = O.make_gptq_case(k, n, m, bits=4, seed=k + n + m + 9, bias=True)
    out = run(M, c, 4, bias=c["bias"], flags=0)
    assert_close(out, oracle_out(c, False, c["bias"]), f"default dispatch {k}x{n} M={m}")
