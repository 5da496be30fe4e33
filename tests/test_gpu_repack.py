"""Load-time transforms through the C ABI: int8 [K,N] -> GPTQ word layout, act-order rows sorted by group,
and the GEMMs that run on the transformed tensors, against the oracle."""
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


def test_w8_pack_is_the_gptq_layout_bit_exact(M):
    c = O.make_w8_case(1024, 384, 1, seed=5)
    qweight, _, _, _ = O.w8_perchannel_as_gptq(c["w"].numpy(), c["scales"])
    packed = M.pack_w8(c["w"].to(DEV))
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), np.asarray(qweight).view(np.uint32))


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("m", [1, 2, 8, 32, 128, 512])
def test_w8linear_runs_packed_on_the_gptq_kernels(M, k, n, m):
    c = O.make_w8_case(k, n, m, seed=m)
    lin = M.W8Linear(k, n)
    lin.update_buffer("weight", c["w"].to(DEV))
    lin.update_buffer("scales", c["scales"].to(DEV))
    out = lin(c["x"].to(DEV))
    assert lin._packed is not None
    assert_close(out, O.w8_perchannel_linear(c["x"], c["w"].numpy(), c["scales"]), f"packed w8 {k}x{n} M={m}")


@pytest.mark.parametrize("bits", [4, 8])
def test_sort_act_order_matches_a_stable_argsort(M, bits):
    c = O.make_gptq_case(2048, 256, 1, bits=bits, act_order=True, seed=9)
    qw, perm = M.sort_act_order(c["qweight"].to(DEV), c["g_idx"].to(DEV), c["scales"].shape[0], bits)
    ref_perm = torch.argsort(c["g_idx"].long(), stable=True).to(torch.int32)
    assert torch.equal(perm.cpu(), ref_perm)
    rows = O.unpack_rows(c["qweight"].numpy(), bits)                 # [K, N] one element per entry
    assert np.array_equal(O.unpack_rows(qw.cpu().numpy(), bits), rows[ref_perm.numpy()])
    # the sorted layer dequantizes (contiguous groups) to the permuted rows of the original
    w_sorted = O.dequantize_packed(qw.cpu(), None, c["qzeros"], c["scales"], bits)
    w_orig = O.dequantize_packed(c["qweight"], c["g_idx"], c["qzeros"], c["scales"], bits)
    assert torch.equal(w_sorted, w_orig[ref_perm.long()])


def test_sort_act_order_rejects_unequal_groups(M):
    c = O.make_gptq_case(1024, 128, 1, bits=4, act_order=True, seed=1)
    g = c["g_idx"].clone()
    g[0] = g[1]                                                        # one group gains a row, another loses one
    if torch.equal(g, c["g_idx"]):
        g[0] = (g[0] + 1) % c["scales"].shape[0]
    with pytest.raises(ValueError):
        M.sort_act_order(c["qweight"].to(DEV), g.to(DEV), c["scales"].shape[0], 4)
    g[0] = 9999
    with pytest.raises(ValueError):
        M.sort_act_order(c["qweight"].to(DEV), g.to(DEV), c["scales"].shape[0], 4)


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 2, 4, 16, 64, 300])
def test_config3_mistral_shapes_act_order_sorted(M, k, n, m):
    c = O.make_gptq_case(k, n, m, bits=4, act_order=True, seed=k + n + m)
    d = to_dev(c, DEV)
    qw, perm = M.sort_act_order(d["qweight"], d["g_idx"], c["scales"].shape[0], 4)
    out = M.quantized_matrix_multiply_ordered(d["x"], qw, d["qzeros"], d["scales"], perm, bits=4)
    assert_close(out, oracle_out(c, True), f"sorted act-order {k}x{n} M={m}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("tune", [1 << 24, 2 << 24])
def test_ordered_gemv_both_schedules(M, dtype, bits, tune):
    c = O.make_gptq_case(2048, 512, 2, bits=bits, act_order=True, dtype=dtype, seed=17, bias=True)
    d = to_dev(c, DEV)
    qw, perm = M.sort_act_order(d["qweight"], d["g_idx"], c["scales"].shape[0], bits)
    out = M.quantized_matrix_multiply_ordered(d["x"], qw, d["qzeros"], d["scales"], perm, bits=bits, bias=d["bias"], flags=16 | tune)
    assert_close(out, oracle_out(c, True, c["bias"]), f"ordered GEMV bits={bits} {dtype}")


def test_qlinear_module_sorts_once_and_matches(M):
    c = O.make_gptq_case(1024, 512, 3, bits=4, act_order=True, seed=23)
    lin = M.QLinear(1024, 512, c["scales"].shape[0], bits=4)
    for name in ("qweight", "qzeros", "scales", "g_idx"):
        lin.update_buffer(name, c[name].to(DEV))
    out = lin(c["x"].to(DEV))
    assert lin._sorted not in (None, False)
    assert_close(out, oracle_out(c, True), "QLinear act-order, M=3 (gather launch)")
    assert_close(lin(c["x"][:1].to(DEV)), oracle_out({**c, "x": c["x"][:1]}, True), "QLinear act-order, M=1 (gather in the GEMV)")
