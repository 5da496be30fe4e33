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
