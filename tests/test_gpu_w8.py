"""mt_w8_perchannel_gemm through the C ABI against the oracle (int8 per-channel = one-group special case)."""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("m", [1, 8, 32, 128, 512])
def test_config2_qwen_shapes(M, k, n, m):
    c = O.make_w8_case(k, n, m, seed=m)
    out = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV))
    assert_close(out, O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"]), f"w8 {k}x{n} M={m}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2, 9, 16, 17, 40, 64])
def test_small_shapes_dtypes_bias(M, dtype, m):
    c = O.make_w8_case(272, 144, m, dtype=dtype, seed=100 + m)
    bias = torch.randn(144, generator=torch.Generator().manual_seed(m)).to(dtype)
    out = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV), bias=bias.to(DEV))
    assert_close(out, O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"], bias), f"w8 {dtype} M={m}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 11008), (11008, 4096), (64, 256), (8192, 512), (272, 768)])
def test_decode_gemv_on_the_plain_layout(M, k, n, m, dtype):
    """M <= 2 and N % 256 == 0 take the CUDA-core GEMV; flags = 1 keeps the mma.sync kernel: both match the oracle."""
    c = O.make_w8_case(k, n, m, dtype=dtype, seed=k + n + m)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(m)).to(dtype)
    ref = O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"], bias)
    for flags in (0, 4, 1):
        out = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV), bias=bias.to(DEV), flags=flags)
        assert_close(out, ref, f"w8 gemv {k}x{n} M={m} {dtype} flags={flags}")


def test_decode_gemv_activation_ranges_and_determinism(M):
    from minit_b200 import _lib
    c = O.make_w8_case(4096, 512, 2, seed=9)
    x = c["x"].float()
    x[:, ::97] *= 200.0
    x[:, 1024:2048] = 0.0
    x[1] *= 2.0 ** -16
    c["x"] = x.half()
    ref = O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"])
    a = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV))
    b = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV))
    assert torch.equal(a, b)
    for row in range(2):                                      # rows differ by 2^16 in magnitude: judge each on its own rms
        assert_close(a[row:row + 1], ref[row:row + 1], f"w8 gemv row {row}")
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


def test_same_result_as_the_gptq_int8_layout(M):
    """The per-channel entry point and mt_qgemm on the equivalent GPTQ-8bit tensors agree."""
    c = O.make_w8_case(1024, 256, 4, seed=3)
    qweight, g_idx, qzeros, s = O.w8_perchannel_as_gptq(c["w"].numpy(), c["scales"])
    a = M.w8_perchannel_matrix_multiply(c["x"].to(DEV), c["w"].to(DEV), c["scales"].to(DEV))
    b = M.quantized_matrix_multiply(c["x"].to(DEV), torch.from_numpy(qweight).to(DEV), torch.from_numpy(qzeros).to(DEV),
                                    s.contiguous().to(DEV), None, bits=8)
    ref = O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"])
    assert_close(a, ref, "per-channel entry")
    assert_close(b, ref, "gptq-int8 entry")
