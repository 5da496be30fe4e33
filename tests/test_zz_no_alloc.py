"""mt_qgemm_static -- the entry point for callers that cannot allocate (a host whose own pool
holds all device memory, or a decode loop that must not touch the allocator) -- called through
the C ABI and compared with mt_qgemm on the same inputs.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It makes two calls in a row (the second finds the library's fixed scratch
array in the state the first left it in) and checks the size limit."""
import ctypes

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


def _static_call(L, d, bits, out, m, n, k, groups, g_idx=None, bias=None):
    """Raw C-ABI call: pointers and sizes only, nothing allocated on the way."""
    stream = torch.cuda.current_stream().cuda_stream
    return L.mt_qgemm_static(stream, d["x"].data_ptr(), d["qweight"].data_ptr(), None if g_idx is None else g_idx.data_ptr(),
                             d["qzeros"].data_ptr(), d["scales"].data_ptr(), None if bias is None else bias.data_ptr(),
                             out.data_ptr(), m, n, k, groups, bits, 0, 0)


@pytest.mark.parametrize("bits,k,n,m,act", [(4, 8192, 2048, 1, False), (4, 4096, 4096, 16, False),
                                            (8, 2048, 1024, 5, False), (4, 1024, 512, 3, True)])
def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(M, bits, k, n, m, act):
    from minit_b200 import _lib
    L = _lib.lib
    c = O.make_gptq_case(k, n, m, bits=bits, act_order=act, seed=k + n + m, bias=True)
    d = to_dev(c, DEV)
    gi = d["g_idx"] if act else None
    ref_entry = M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"], d["scales"], gi, bits=bits,
                                            bias=d["bias"], flags=_lib.FLAG_FORCE_SMALL)
    oracle = oracle_out(c, act, c["bias"])
    out = torch.empty((m, n), dtype=torch.float16, device=DEV)
    for attempt in range(2):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _static_call(L, d, bits, out, m, n, k, k // 128, gi, d["bias"])
        assert rc == 0, L.mt_strerror(rc).decode()
        torch.cuda.synchronize()
        if attempt == 1:   # warmed up: the call itself must not have taken any device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        # same tolerance as every other GEMM test: max|a - b| <= 1e-2 * rms
        assert_close(out, ref_entry.cpu(), f"static vs workspace entry, call {attempt}")
        assert_close(out, oracle, f"static entry vs oracle, call {attempt}")


def test_static_scratch_entry_python_wrapper_and_limit(M):
    from minit_b200 import _lib
    c = O.make_gptq_case(512, 256, 2, bits=4, seed=1)
    d = to_dev(c, DEV)
    out = torch.empty((2, 256), dtype=torch.float16, device=DEV)
    M.quantized_matrix_multiply_noalloc(d["x"], d["qweight"], d["qzeros"], d["scales"], None, out, bits=4)
    assert_close(out, oracle_out(c, False), "python wrapper")
    # beyond the fixed array: K = 8192, N = 57344 needs ~44 MB of split-K scratch -> refused up front
    a = 1 << 20
    rc = _lib.lib.mt_qgemm_static(None, a, a, None, a, a, None, a, 1, 57344, 8192, 64, 4, 0, 0)
    assert rc == -10
    assert b"capacity" in _lib.lib.mt_strerror(rc)
    assert _lib.lib.mt_workspace_bytes(1, 8192, 8192, 4) <= _lib.STATIC_SCRATCH_BYTES


_FRESH = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
from oracle import qlinear_oracle as O
from minit_b200 import _lib
c = O.make_gptq_case(1024, 512, 2, bits=4, seed=3)
d = {k: (v.to("cuda:0") if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
out = torch.empty((2, 512), dtype=torch.float16, device="cuda:0")
torch.cuda.synchronize()
free = [torch.cuda.mem_get_info()[0]]
for _ in range(2):
    rc = _lib.lib.mt_qgemm_static(torch.cuda.current_stream().cuda_stream, d["x"].data_ptr(), d["qweight"].data_ptr(), None,
                                  d["qzeros"].data_ptr(), d["scales"].data_ptr(), None, out.data_ptr(), 2, 512, 1024, 8, 4, 0, 0)
    torch.cuda.synchronize()
    free.append(torch.cuda.mem_get_info()[0])
ref = O.qlinear(c["x"], O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4))
ok, err, bound = O.tolerance_ok(out, ref, 1e-2)
print(json.dumps({"rc": rc, "first_call_took": free[0] - free[1], "second_call_took": free[1] - free[2], "ok": bool(ok)}))
"""


def test_static_scratch_first_call_in_a_fresh_process(lib_built):
    """The documented cost of the very first call on a device: with lazy module loading it is the call that makes
    the driver load the module holding the fixed array (so it may take device memory, once); every later call
    takes none.  A fresh process, so that no earlier test has already loaded that module."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _FRESH, root], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["rc"] == 0 and rec["ok"], rec
    assert rec["second_call_took"] == 0, rec
    # first call: nothing (module already resident, e.g. eager loading) or a one-time reservation of a few MiB
    # (the 8 MiB array plus the module's code, in the driver's allocation granularity)
    assert 0 <= rec["first_call_took"] <= 256 << 20, rec
    print("first mt_qgemm_static call on the device took", rec["first_call_took"], "bytes of device memory")
