"""``matrix_multiply(x, QuantizedTensor)`` and ``dispatch(MatrixMultiply(), x, qt)`` (reference:
minit/functional/linalg.py:9-20, minit/quantize/dispatch.py:8-11, the ``weight`` property at
examples/qwen1_5_int8.py:283-285) against the oracle, for a packed and an unpacked operand, 2-D and folded."""
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


def _qlinear(M, c, bits, dtype):
    k, n = c["q"].shape
    lin = M.QLinear(k, n, c["scales"].shape[0], bits=bits, dtype=str(dtype).replace("torch.", ""))
    d = to_dev(c, DEV)
    for name in ("qweight", "qzeros", "scales", "g_idx"):
        lin.update_buffer(name, d[name])
    return lin, d


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("act_order", [False, True])
@pytest.mark.parametrize("lead", [(3,), (2, 5), (1,)])
def test_matrix_multiply_with_qlinear_weight(M, bits, act_order, lead):
    m = 1
    for v in lead:
        m *= v
    c = O.make_gptq_case(512, 384, m, bits=bits, act_order=act_order, seed=11 + bits + m)
    lin, d = _qlinear(M, c, bits, torch.float16)
    x = d["x"].reshape(*lead, 512)
    out = M.matrix_multiply(x, lin.weight)                      # packed operand: the fused kernel
    assert tuple(out.shape) == (*lead, 384)
    ref = oracle_out(c, act_order)
    assert_close(out.reshape(m, 384), ref, f"matrix_multiply packed bits={bits} act={act_order} lead={lead}")
    (out2,) = M.dispatch(M.MatrixMultiply(), d["x"], lin.weight)
    assert torch.equal(out2, out.reshape(m, 384))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_matrix_multiply_with_unpacked_operand(M, bits, dtype):
    """QuantizedTensor(data, group, zero, scale) as the reference constructs it: one element per byte."""
    c = O.make_gptq_case(256, 128, 6, bits=bits, act_order=True, dtype=dtype, seed=5 + bits)
    d = to_dev(c, DEV)
    qt = M.QuantizedTensor(torch.from_numpy(c["q"]).to(DEV), d["g_idx"], torch.from_numpy(c["z"]).to(DEV), d["scales"])
    assert qt.packed is None and tuple(qt.shape) == (256, 128)
    ref = oracle_out(c, True)
    (out,) = M.dispatch(M.MatrixMultiply(), d["x"], qt)
    assert_close(out, ref, f"dispatch unpacked bits={bits} {dtype}")
    out3 = M.matrix_multiply(d["x"].reshape(2, 3, 256), qt)
    assert tuple(out3.shape) == (2, 3, 128)
    assert torch.equal(out3.reshape(6, 128), out)
    # the unpacked operand dequantizes to the oracle's W bit for bit
    w = qt.dequantize()
    assert torch.equal(w.cpu().view(torch.int16), O.dequantize(c["q"], c["g_idx"].numpy(), c["z"], c["scales"]).view(torch.int16))


def test_dispatch_rejects_unknown_operands(M):
    with pytest.raises(TypeError):
        M.dispatch(M.MatrixMultiply(), torch.zeros(2, 2, device=DEV), "not a tensor")
