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
        res = torch.randn((4, 1024), generator=torch.Generator().manual_seed(5)).half()
        yr = row(h_local * 0.05, residual=res.to(dev))  # NCCL path: rank 0 folds the residual into its partial
        ok, err, bound = O.tolerance_ok(yr, O.add_residual(res, ref), 2e-2)
        assert ok, f"rank {rank} residual over NCCL: err {err} > {bound}"
        # the same row-parallel linear with the all-reduce fused into the GEMM epilogue (peer memory, no NCCL):
        # several calls in a row (alternating slots), two shapes, bit-identical on all ranks
        from minit_b200.collective import FusedAllReduce
        far = FusedAllReduce(m_max=16, n_max=4096)
        far8k = FusedAllReduce(m_max=2, n_max=8192)
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
        # decode shapes (M = 1, 2) take the CUDA-core GEMV, both schedules; N = 8192 crosses many column blocks
        for m4, seed4, tune in [(1, 41, 0), (2, 42, 1 << 24), (2, 43, 2 << 24), (1, 44, 2 << 24)]:
            c4 = O.make_gptq_case(4096, 8192, m4, bits=4, seed=seed4, bias=True)
            rowf4 = RowParallelQLinear(comm, g(c4, "qweight"), g(c4, "qzeros"), g(c4, "scales"), None, 4, bias=g(c4, "bias"), fused=far8k)
            ks4 = 4096 // size
            x4 = g(c4, "x")[:, ks4 * rank:ks4 * (rank + 1)].contiguous()
            ref4 = O.qlinear(c4["x"], O.dequantize_packed(c4["qweight"], None, c4["qzeros"], c4["scales"], 4), c4["bias"])
            for it in range(3):
                y4 = rowf4(x4, flags=tune)
                ok, err, bound = O.tolerance_ok(y4, ref4, 1e-2)
                assert ok, f"rank {rank} fused GEMV M={m4} tune={tune:#x} call {it}: err {err} > {bound}"
            g4 = [torch.empty_like(y4) for _ in range(size)]
            dist.all_gather(g4, y4)
            assert all(torch.equal(g4[0], t) for t in g4), "fused GEMV all-reduce results differ between ranks"
            # the block's residual add folded into the same kernel (added once, to the reduced sum)
            res4 = torch.randn((m4, 8192), generator=torch.Generator().manual_seed(seed4)).half()
            y4r = rowf4(x4, flags=tune, residual=res4.to(dev))
            ok, err, bound = O.tolerance_ok(y4r, O.add_residual(res4, ref4), 1e-2)
            assert ok, f"rank {rank} fused GEMV + residual M={m4} tune={tune:#x}: err {err} > {bound}"
        # batches of 8 and 32 rows on a weight large enough for the integer tensor-core kernel: the same exchange in its epilogue
        # (one value per thread), residual added after the reduction, identical on all ranks, replayable from a graph
        far32 = FusedAllReduce(m_max=32, n_max=8192)
        MID = 128                                            # MT_FLAG_FORCE_MID: the integer kernel whatever the size rule says
        for m5, seed5 in [(8, 51), (32, 52), (5, 53)]:
            c5 = O.make_gptq_case(8192, 8192, m5, bits=4, seed=seed5, bias=True)
            rowf5 = RowParallelQLinear(comm, g(c5, "qweight"), g(c5, "qzeros"), g(c5, "scales"), None, 4, bias=g(c5, "bias"), fused=far32)
            ks5 = 8192 // size
            x5 = g(c5, "x")[:, ks5 * rank:ks5 * (rank + 1)].contiguous()
            sl = slice(3000, 3512)
            w5 = O.dequantize_packed(c5["qweight"][:, sl].contiguous(), None, c5["qzeros"][:, sl.start // 8:sl.stop // 8].contiguous(),
                                     c5["scales"][:, sl].contiguous(), 4)
            ref5 = O.qlinear(c5["x"], w5, c5["bias"][sl])
            for it in range(3):
                y5 = rowf5(x5, flags=MID)
                ok, err, bound = O.tolerance_ok(y5[:, sl], ref5, 1e-2)
                assert ok, f"rank {rank} fused integer kernel M={m5} call {it}: err {err} > {bound}"
            g5 = [torch.empty_like(y5) for _ in range(size)]
            dist.all_gather(g5, y5)
            assert all(torch.equal(g5[0], t) for t in g5), "fused integer-kernel all-reduce results differ between ranks"
            # the two-shot exchange (partials to the column's owner rank, the sum back; by flag): the
            # owner adds in the same rank order, so the result has the same bits; one-shot and two-shot calls alternate
            TWO = 1024                                       # MT_FLAG_AR_TWO_SHOT
            for it in range(3):
                y5t = rowf5(x5, flags=MID | TWO)
                assert torch.equal(y5t, y5), f"rank {rank} two-shot exchange differs from the one-shot one (M={m5}, call {it})"
                assert torch.equal(rowf5(x5, flags=MID), y5)
            g5t = [torch.empty_like(y5t) for _ in range(size)]
            dist.all_gather(g5t, y5t)
            assert all(torch.equal(g5t[0], t) for t in g5t), "two-shot all-reduce results differ between ranks"
            res5 = torch.randn((m5, 8192), generator=torch.Generator().manual_seed(seed5)).half()
            y5r = rowf5(x5, flags=MID, residual=res5.to(dev))
            ok, err, bound = O.tolerance_ok(y5r[:, sl], O.add_residual(res5[:, sl], ref5), 1e-2)
            assert ok, f"rank {rank} fused integer kernel + residual M={m5}: err {err} > {bound}"
        y5g = torch.empty_like(y5)
        side5 = torch.cuda.Stream()
        side5.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side5):
            rowf5(x5, out=y5g, flags=MID)
            torch.cuda.synchronize()
            graph5 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph5, stream=side5):
                rowf5(x5, out=y5g, flags=MID)
                rowf5(x5, out=y5g, flags=MID)
            for _ in range(3):
                graph5.replay()
            torch.cuda.synchronize()
        torch.cuda.current_stream().wait_stream(side5)
        assert torch.equal(y5g, y5), "graph replay of the fused integer kernel differs from the eager call"
        # a captured graph of fused calls replays correctly: the call counter lives on the device
        xg = x4.clone(); yg = torch.empty_like(y4)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            rowf4(xg, out=yg); rowf3(x3)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                rowf4(xg, out=yg)
                rowf4(xg, out=yg)
                rowf4(xg, out=yg)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
        ok, err, bound = O.tolerance_ok(yg, ref4, 1e-2)
        assert ok, f"rank {rank} graph replay of the fused GEMV: err {err} > {bound}"
        torch.cuda.current_stream().wait_stream(side)
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
