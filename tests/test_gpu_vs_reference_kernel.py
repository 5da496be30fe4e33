"""Our kernels beside the reference's OWN fused kernel on the same GPU and inputs.  The reference kernel
(examples/qwen1_5_int8.py:156-216, 8-bit only) is built unchanged from its source string by
oracle/build_ref_cuda.py into oracle/_ref/ (not tracked; it travels with the working tree); without that library the
tests are skipped.  The reference adds fp16-rounded partial sums of 32 values of k with atomicAdd, so it is the less
exact of the two: at K = 4096 it sits outside the north-star bound against the oracle on its own."""
import ctypes
import os

import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIB = os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "libref_qmm_f16.so")


@pytest.fixture(scope="module")
def ref_qmm():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libref_qmm_f16.so is not built (needs a checkout of the reference: oracle/build_ref_cuda.py)")
    fn = ctypes.CDLL(LIB).qmm_ref
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.restype, fn.argtypes = None, [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci]
    return fn


@pytest.mark.parametrize("k,n,m,gs,act", [(512, 256, 1, 128, False), (1024, 512, 2, 64, True), (1024, 2048, 16, 128, False), (4096, 4096, 1, 128, False)])
def test_same_inputs_as_the_reference_kernel(lib_built, ref_qmm, k, n, m, gs, act):
    import minit_b200 as M
    c = O.make_gptq_case(k, n, m, bits=8, group_size=gs, act_order=act, seed=k + n + m)
    d = to_dev(c, DEV)
    theirs = torch.zeros((m, n), dtype=torch.float16, device=DEV)            # the reference's wrapper zeroes the output first
    ref_qmm(None, d["x"].data_ptr(), d["qweight"].data_ptr(), d["g_idx"].data_ptr(), d["qzeros"].data_ptr(), d["scales"].data_ptr(),
            theirs.data_ptr(), m, n, k, k // gs)
    ours = M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"], d["scales"], d["g_idx"] if act else None, bits=8)
    torch.cuda.synchronize()
    exact = oracle_out(c, act)
    ok, e_ours, bound = O.tolerance_ok(ours.cpu(), exact, 1e-2)
    assert ok, f"{k}x{n} M={m}: |ours - oracle| = {e_ours} > {bound}"
    # the reference kernel rounds to fp16 at each of its K / 32 atomic adds: it stays within 2.5e-2 * rms of the contract
    ok, e_theirs, bound_t = O.tolerance_ok(theirs.cpu(), exact, 2.5e-2)
    assert ok, f"{k}x{n} M={m}: |reference kernel - oracle| = {e_theirs} > {bound_t}"
    # so the two agree to the sum of their distances from it, and ours is the closer one
    diff = (ours.cpu().float() - theirs.cpu().float()).abs().max().item()
    assert diff <= e_ours + e_theirs + 1e-6
    assert e_ours <= e_theirs + 1e-3, f"ours is further from the oracle ({e_ours}) than the reference kernel ({e_theirs})"
