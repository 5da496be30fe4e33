"""Tensor-parallel quantized linears on real GPUs over NCCL (skipped with fewer than 2 GPUs):
column-parallel -> row-parallel -> in-place all-reduce equals the unsharded oracle."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, size, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=size, device_id=torch.device("cuda", rank))
    try:
        from oracle import qlinear_oracle as O
        from minit_b200.collective import ColumnParallelQLinear, RowParallelQLinear
        from minit_b200.distributed import DistributedCommunicator, initialize_world
        from minit_b200.nccl import NCCLTensor
        from minit_b200.nccl.library import exchange_unique_id
        initialize_world(rank, size)
        comm = DistributedCommunicator(NCCLTensor.connect(exchange_unique_id(rank), rank, size, device=rank))
        dev = f"cuda:{rank}"
        c1 = O.make_gptq_case(1024, 2048, 4, bits=4, seed=1)               # column-parallel (gate/up-like)
        c2 = O.make_gptq_case(2048, 1024, 4, bits=4, seed=2, bias=True)    # row-parallel (down-like)
        g = lambda c, k: c[k].to(dev)
        col = ColumnParallelQLinear(g(c1, "qweight"), g(c1, "qzeros"), g(c1, "scales"), None, 4)
        row = RowParallelQLinear(comm, g(c2, "qweight"), g(c2, "qzeros"), g(c2, "scales"), None, 4, bias=g(c2, "bias"))
        h_local = col(g(c1, "x"))                       # [4, 2048/size], stays sharded
        y = row(h_local * 0.05)                         # partial [4,1024] summed in place over NCCL
        w1 = O.dequantize_packed(c1["qweight"], None, c1["qzeros"], c1["scales"], 4)
        w2 = O.dequantize_packed(c2["qweight"], None, c2["qzeros"], c2["scales"], 4)
        h = O.qlinear(c1["x"], w1) * 0.05
        ref = O.qlinear(h, w2, c2["bias"])
        ok, err, bound = O.tolerance_ok(y, ref, 2e-2)   # two chained linears + fp16 all-reduce: 2e-2 * rms
        assert ok, f"rank {rank}: err {err} > {bound}"
        # the same row-parallel linear with the all-reduce fused into the GEMM epilogue (peer memory, no NCCL):
        # several calls in a row (alternating slots), two shapes, bit-identical on all ranks
        from minit_b200.collective import FusedAllReduce
        far = FusedAllReduce(m_max=16, n_max=4096)
        rowf = RowParallelQLinear(comm, g(c2, "qweight"), g(c2, "qzeros"), g(c2, "scales"), None, 4, bias=g(c2, "bias"), fused=far)
        c3 = O.make_gptq_case(8192, 512, 1, bits=4, seed=3)
        rowf3 = RowParallelQLinear(comm, g(c3, "qweight"), g(c3, "qzeros"), g(c3, "scales"), None, 4, fused=far)
        ks3 = 8192 // size
        x3 = g(c3, "x")[:, ks3 * rank:ks3 * (rank + 1)].contiguous()
        ref3 = O.qlinear(c3["x"], O.dequantize_packed(c3["qweight"], None, c3["qzeros"], c3["scales"], 4))
        for it in range(5):
            yf = rowf(h_local * 0.05)
            ok, err, bound = O.tolerance_ok(yf, ref, 2e-2)
            assert ok, f"rank {rank} fused call {it}: err {err} > {bound}"
            y3 = rowf3(x3)
            ok, err, bound = O.tolerance_ok(y3, ref3, 1e-2)
            assert ok, f"rank {rank} fused (split-K) call {it}: err {err} > {bound}"
        gathered = [torch.empty_like(y3) for _ in range(size)]
        dist.all_gather(gathered, y3)
        assert all(torch.equal(gathered[0], t) for t in gathered), "fused all-reduce results differ between ranks"
        from minit_b200 import _lib
        torch.cuda.synchronize()
        for ws in _lib._workspaces.values():
            assert _lib.workspace_error_word(ws) == 0, "a bounded wait of the fused all-reduce expired"
        # the three collectives of the communicator
        t = torch.full((4, 8), float(rank + 1), device=dev, dtype=torch.float16)
        assert torch.equal(comm.all_reduce(t), torch.full_like(t, float(sum(range(1, size + 1)))))
        ga = comm.all_gather(t[:, :2].contiguous(), 1)
        assert ga.shape == (4, 2 * size) and float(ga[0, -1]) == float(size)
        assert torch.equal(comm.broadcast(t, 1), torch.full_like(t, 2.0))
        torch.cuda.synchronize()
        results[rank] = "ok"
    except BaseException as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(type(e), e, e.__traceback__))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_column_then_row_parallel_over_nccl(lib_built):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    size = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(size, _free_port(), results), nprocs=size, join=True)
        for r in range(size):
            assert results.get(r) == "ok", f"rank {r}: {results.get(r)}"
