"""mt_dequant / mt_dequant_unpacked / mt_unpack through the C ABI against the golden vectors and the oracle: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.test_oracle import CASES, GOLDEN, load_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


@pytest.mark.parametrize("name", CASES)
def test_dequant_matches_golden_bit_exactly(M, name):
    from minit_b200.quantize.tensor import dequantize_packed
    c = load_case(np.load(GOLDEN), name)
    qw = torch.from_numpy(c["qweight"]).to(DEV)
    qz = torch.from_numpy(c["qzeros"]).to(DEV)
    gi = torch.from_numpy(c["g_idx"]).to(DEV)
    w = dequantize_packed(qw, gi, qz, c["scales"].to(DEV), c["bits"])
    assert np.array_equal(w.cpu().view(torch.int16).numpy(), c["w_bits"])
    # the unpacked route the reference's QuantizedTensor takes
    qt = M.QuantizedTensor(M.unpack(qw, 0, c["bits"]), gi, M.unpack(qz, 1, c["bits"]), c["scales"].to(DEV))
    assert np.array_equal(qt.dequantize().cpu().view(torch.int16).numpy(), c["w_bits"])
    assert np.array_equal(M.unpack(qw, 0, c["bits"]).cpu().numpy(), O.unpack_rows(c["qweight"], c["bits"]))
    assert np.array_equal(M.unpack(qz, 1, c["bits"]).cpu().numpy(), O.unpack_cols(c["qzeros"], c["bits"]))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", [False, True])
def test_dequant_matches_oracle_bit_exactly(M, bits, dtype, act):
    from minit_b200.quantize.tensor import dequantize_packed
    c = O.make_gptq_case(1024, 512, 1, bits=bits, act_order=act, dtype=dtype, seed=3)
    ref = O.dequantize_packed(c["qweight"], c["g_idx"] if act else None, c["qzeros"], c["scales"], bits)
    w = dequantize_packed(c["qweight"].to(DEV), c["g_idx"].to(DEV) if act else None, c["qzeros"].to(DEV),
                          c["scales"].to(DEV), bits)
    assert torch.equal(w.cpu().view(torch.int16), ref.view(torch.int16))


def test_dequant_every_q_z_pair_and_null_zeros(M):
    """All 16x16 (q, z) nibble pairs and all 256x256 byte pairs, plus the NULL-zeros midpoint."""
    from minit_b200.quantize.tensor import dequantize_packed
    for bits in (4, 8):
        lv = 1 << bits
        k, n = (lv * 32 // 32) * 32, lv if lv >= 8 else 8
        k = max(32, lv)          # q value = k index mod levels
        k = ((k + 31) // 32) * 32
        q = (np.arange(k)[:, None] % lv).astype(np.uint8).repeat(n, 1)
        z = (np.arange(n)[None, :] % lv).astype(np.uint8)
        scales = (0.001 + 0.02 * torch.rand((1, n), generator=torch.Generator().manual_seed(bits))).half()
        qw, qz = torch.from_numpy(O.pack_rows(q, bits)), torch.from_numpy(O.pack_cols(z, bits))
        ref = O.dequantize(q, np.zeros(k, np.int32), z, scales)
        w = dequantize_packed(qw.to(DEV), None, qz.to(DEV), scales.to(DEV), bits)
        assert torch.equal(w.cpu().view(torch.int16), ref.view(torch.int16))
        ref0 = O.dequantize_packed(qw, None, None, scales, bits)
        w0 = dequantize_packed(qw.to(DEV), None, None, scales.to(DEV), bits)
        assert torch.equal(w0.cpu().view(torch.int16), ref0.view(torch.int16))


def test_dequant_full_size_config1_roundtrip_property(M):
    """K = N = 4096 (the full single-linear config): bit-exact against the oracle, and
    dequantizing with scale 1 / zero such that z+1 = 0 is impossible, so use linearity in the
    scale instead: W(2s) == 2 * W(s) exactly (power-of-two scaling commutes with rounding)."""
    from minit_b200.quantize.tensor import dequantize_packed
    c = O.make_gptq_case(4096, 4096, 1, bits=4, seed=0)
    d = {k: v.to(DEV) for k, v in c.items() if isinstance(v, torch.Tensor)}
    w = dequantize_packed(d["qweight"], None, d["qzeros"], d["scales"], 4)
    ref = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4)
    assert torch.equal(w.cpu().view(torch.int16), ref.view(torch.int16))
    w2 = dequantize_packed(d["qweight"], None, d["qzeros"], d["scales"] * 2, 4)
    assert torch.equal(w2, w * 2)


@pytest.mark.parametrize("name", ["unpack_a", "unpack_b"])
def test_unpack_matches_the_reference_unpack(M, name):
    """mt_unpack against the bytes the reference's own unpack() produced (tests/golden/make_golden.py)."""
    g = np.load(GOLDEN)
    x = torch.from_numpy(g[f"{name}.x"]).to(DEV)
    assert np.array_equal(M.unpack(x, 0, 8).cpu().numpy(), g[f"{name}.axis0"])
    assert np.array_equal(M.unpack(x, 1, 8).cpu().numpy(), g[f"{name}.axis1"])
