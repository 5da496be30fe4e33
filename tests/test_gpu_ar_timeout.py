"""The time-out path of the fused GEMM + all-reduce, exercised without a second GPU and without a fault: a "world" of
two symmetric buffers that both live on this GPU, of which only rank 0 ever launches.  Its wait for rank 1's values runs
out (MT_FLAG_AR_SHORT_WAIT keeps that to a fraction of a millisecond), the kernel returns normally, the workspace error
word reads 4 and the host-side check raises.  The context stays usable: the same entry point with world = 1 then
reproduces the oracle."""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("m,force_small,k,n", [(1, False, 1024, 512), (2, False, 1024, 512), (4, True, 1024, 512),
                                               (8, False, 4096, 8192)])     # the last one: the integer tensor-core kernel
def test_expired_peer_wait_sets_the_error_word_and_raises(lib_built, m, force_small, k, n):
    from minit_b200 import _lib
    L = _lib.lib
    c = O.make_gptq_case(k, n, m, bits=4, seed=40 + m)
    d = to_dev(c, DEV)
    dev = torch.device(DEV)
    nbytes = int(L.mt_allreduce_buffer_bytes(m, n, 2))
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    stream = _lib.current_stream(dev)
    ws = _lib.workspace(dev, stream, L.mt_workspace_bytes(m, n, k, 4))
    _lib.raise_on_error_words()                                   # clean before the experiment
    flags = _lib.FLAG_AR_SHORT_WAIT | (_lib.FLAG_FORCE_SMALL if force_small else 0) | (_lib.FLAG_FORCE_MID if m == 8 else 0)
    rc = L.mt_qgemm_allreduce(stream, d["x"].data_ptr(), d["qweight"].data_ptr(), None, d["qzeros"].data_ptr(),
                              d["scales"].data_ptr(), None, out.data_ptr(), m, n, k, k // 128, 4, 0, ws.data_ptr(), ws.numel(),
                              flags, table.data_ptr(), 0, 2, nbytes)
    assert rc == 0
    torch.cuda.synchronize()                                      # the kernel returned by itself
    assert _lib.workspace_error_word(ws) == 4
    with pytest.raises(_lib.MinitError) as info:
        _lib.raise_on_error_words()
    assert info.value.status == _lib.ERR_PEER_TIMEOUT
    assert _lib.workspace_error_word(ws) == 0                     # the check cleared it
    # the context and the workspace are still good
    rc = L.mt_qgemm_allreduce(stream, d["x"].data_ptr(), d["qweight"].data_ptr(), None, d["qzeros"].data_ptr(),
                              d["scales"].data_ptr(), None, out.data_ptr(), m, n, k, k // 128, 4, 0, ws.data_ptr(), ws.numel(),
                              flags, None, 0, 1, 0)
    assert rc == 0
    torch.cuda.synchronize()
    assert_close(out, oracle_out(c, False), "world 1 after the expired wait")
    _lib.raise_on_error_words()
