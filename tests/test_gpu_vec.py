"""Parity of the CUDA-core decode GEMV (M <= 2, MT_FLAG_FORCE_VEC) with the oracle, through the C ABI.

The kernel multiplies the packed integers as fp16 subnormals against block-scaled activations and
folds scale and zero point per chunk in fp32, so besides the usual shapes the cases cover what that
scheme is sensitive to: activations with outliers, tiny and huge magnitudes, every fold chunk size,
ragged warp runs (forced split-K factors) and bf16 activations.
"""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200

VEC = 16
# tuning field of the flags (bits 24-27): 0 = the library chooses, 1 = one CTA per (column block, split),
# 2 = stream-K schedule
VARIANTS = [0, 1 << 24, 2 << 24]


def splits_flag(s):
    return (s & 0xff) << 16


@pytest.fixture(params=VARIANTS, ids=["auto", "split", "stream"])
def variant(request):
    return request.param


def run(M, c, bits, bias=None, flags=VEC, zeros=True):
    d = to_dev(c, DEV)
    return M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"] if zeros else None, d["scales"], None,
                                       bits=bits, bias=None if bias is None else bias.to(DEV), flags=flags)


def ref(c, bits, bias=None, zeros=True):
    w = O.dequantize_packed(c["qweight"], None, c["qzeros"] if zeros else None, c["scales"], bits)
    return O.qlinear(c["x"], w, bias)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("k,n", [(1024, 768), (4096, 4096), (8192, 512), (256, 128)])
def test_shapes_dtypes(M, variant, bits, dtype, m, k, n):
    c = O.make_gptq_case(k, n, m, bits=bits, dtype=dtype, seed=k + n + m)
    assert_close(run(M, c, bits, flags=VEC | variant), ref(c, bits), f"vec bits={bits} {dtype} M={m} {k}x{n}")


@pytest.mark.parametrize("gs", [32, 64, 96, 128, 256, 1024])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 2])
def test_group_sizes(M, variant, gs, bits, m):
    k = 3072 if gs == 96 else 2048
    c = O.make_gptq_case(k, 256, m, bits=bits, group_size=gs, seed=gs + m)
    assert_close(run(M, c, bits, flags=VEC | variant), ref(c, bits), f"vec group {gs} bits {bits}")


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 7])
@pytest.mark.parametrize("k,gs", [(2080, 32), (4160, 64), (8192, 128)])
def test_ragged_warp_runs(M, variant, splits, k, gs):
    """Chunk counts that do not divide by splits * 8: warp runs of unequal length, odd chunk counts."""
    c = O.make_gptq_case(k, 384, 2, bits=4, group_size=gs, seed=k + splits)
    assert_close(run(M, c, 4, flags=VEC | variant | splits_flag(splits)), ref(c, 4), f"vec splits={splits} K={k}")


def test_bias_null_zeros_overwrite(M, variant):
    c = O.make_gptq_case(2048, 256, 2, bits=4, seed=77, bias=True)
    assert_close(run(M, c, 4, bias=c["bias"], flags=VEC | variant), ref(c, 4, c["bias"]), "vec bias")
    d = to_dev(c, DEV)
    buf = torch.full((2, 256), 1000.0, dtype=torch.float16, device=DEV)
    M.quantized_matrix_multiply(d["x"], d["qweight"], None, d["scales"], None, bits=4, out=buf, flags=VEC | variant)
    assert_close(buf, ref(c, 4, zeros=False), "vec null zeros / overwrite")
    c8 = O.make_gptq_case(2048, 256, 1, bits=8, seed=78, bias=True)
    assert_close(run(M, c8, 8, bias=c8["bias"], zeros=False, flags=VEC | variant), ref(c8, 8, c8["bias"], zeros=False), "vec int8 null zeros")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind", ["outliers", "tiny", "huge", "zeros", "one_hot"])
def test_activation_ranges(M, variant, dtype, kind):
    """Block scaling of the activations: per-chunk maxima far apart, subnormal fp16 inputs, values near the
    top of the fp16 range, all-zero chunks."""
    c = O.make_gptq_case(4096, 256, 2, bits=4, dtype=dtype, seed=91)
    x = c["x"].float()
    if kind == "outliers":
        x[:, ::257] *= 300.0
    elif kind == "tiny":
        x *= 2.0 ** -18
    elif kind == "huge":
        x *= 2000.0
    elif kind == "zeros":
        x[:, 512:2048] = 0.0
    else:
        x.zero_(); x[0, 1234] = 1.0; x[1, 7] = -3.0
    c["x"] = x.to(dtype)
    assert_close(run(M, c, 4, flags=VEC | variant), ref(c, 4), f"vec activations {kind} {dtype}")


def test_deterministic_pdl_and_workspace_left_clean(M, variant):
    from minit_b200 import _lib
    c = O.make_gptq_case(8192, 512, 2, bits=4, seed=4)
    a = run(M, c, 4, flags=VEC | variant)
    for _ in range(3):
        b = run(M, c, 4, flags=VEC | variant | 4)
    assert torch.equal(a, b)
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


def test_wide_and_deep_shapes_cross_column_blocks(M, variant):
    """Runs of the stream-K schedules that start in one column block and end in the next, and blocks
    shared by many warps."""
    for k, n, m in [(512, 4096, 1), (16384, 128, 2), (1024, 2048, 2), (64, 1024, 1)]:
        c = O.make_gptq_case(k, n, m, bits=4, group_size=64, seed=k + n)
        assert_close(run(M, c, 4, flags=VEC | variant), ref(c, 4), f"vec {k}x{n} M={m}")


def test_decode_plan_reports_the_schedule(M):
    """mt_decode_plan: > 0 split-K factor, 0 stream-K, negative status when the GEMV does not take the call."""
    from minit_b200 import _lib
    L = _lib.lib
    ws = lambda m, n, k: L.mt_workspace_bytes(m, n, k, 4)
    assert L.mt_decode_plan(1, 8192, 8192, 64, 4, ws(1, 8192, 8192), 0) == 4            # 64 column blocks x 4 = one wave
    assert L.mt_decode_plan(1, 10240, 8192, 64, 4, ws(1, 10240, 8192), 0) == 3
    assert L.mt_decode_plan(1, 57344, 8192, 64, 4, ws(1, 57344, 8192), 0) in (0, 1)     # 448 blocks: stream-K ties with one split
    assert L.mt_decode_plan(1, 57344, 28672, 224, 4, ws(1, 57344, 28672), 0) == 0        # far more blocks than slots: stream-K
    assert L.mt_decode_plan(1, 8192, 8192, 64, 4, ws(1, 8192, 8192), 2 << 24) == 0       # forced stream-K
    assert L.mt_decode_plan(1, 8192, 8192, 64, 4, ws(1, 8192, 8192), (1 << 24) | (5 << 16)) == 5
    assert L.mt_decode_plan(3, 8192, 8192, 64, 4, ws(3, 8192, 8192), 0) < 0              # M > 2: another kernel
    assert L.mt_decode_plan(1, 136, 1024, 8, 4, ws(1, 136, 1024), 0) < 0                 # N % 128 != 0


def test_unsupported_shapes_are_refused(M):
    c = O.make_gptq_case(1024, 136, 1, bits=4, seed=2)       # N not a multiple of 128
    with pytest.raises(RuntimeError):
        run(M, c, 4)
    c = O.make_gptq_case(1024, 128, 3, bits=4, seed=2)       # M > 2
    with pytest.raises(RuntimeError):
        run(M, c, 4)
