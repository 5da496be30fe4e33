"""Tensor-parallel host logic on two CPU ranks (gloo): shard helpers, CollectiveTensor
conversions and the column-/row-parallel rules.  The local matmul a rank runs here is the
oracle's (there is no CPU kernel in the package); what is under test is the sharding and
where the all-reduce goes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, size, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        from oracle import qlinear_oracle as O
        import minit_b200.collective.quantized as Q
        from minit_b200.collective import (CollectiveTensor, ColumnParallelQLinear, RowParallelQLinear,
                                           shard_gptq_column, shard_gptq_row)
        from minit_b200.collective.spec import CollectiveSpecPartial, CollectiveSpecSplit
        from minit_b200.distributed import DistributedCommunicator, initialize_world
        from minit_b200.distributed.torchdist import TorchDistTensor
        from minit_b200.functional.linalg import matrix_multiply

        initialize_world(rank, size)
        comm = DistributedCommunicator(TorchDistTensor())

        # CPU ranks have no kernel: the local product of a shard is the oracle's
        def cpu_qmm(x, qweight, zeros, scales, groups, *, bits=8, bias=None, out=None, flags=0):
            w = O.dequantize_packed(qweight, groups, zeros, scales, bits)
            return O.qlinear(x, w, bias)
        Q.quantized_matrix_multiply = cpu_qmm

        c = O.make_gptq_case(512, 128, 4, bits=4, seed=42, bias=True)
        w_full = O.dequantize_packed(c["qweight"], None, c["qzeros"], c["scales"], 4)
        ref = c["x"].float() @ w_full.float()

        # 1. collectives and conversions
        t = torch.full((2, 3), float(rank + 1))
        assert torch.equal(comm.all_reduce(t), torch.full((2, 3), float(sum(range(1, size + 1)))))
        g = comm.all_gather(torch.full((2, 1), float(rank)), 1)
        assert g.shape == (2, size) and g[0].tolist() == [float(r) for r in range(size)]
        assert torch.equal(comm.broadcast(torch.full((2,), float(rank)), 1), torch.full((2,), 1.0))
        full = CollectiveTensor.from_broadcast(comm, c["x"])
        sp = full.to_split(1)
        assert isinstance(sp.spec, CollectiveSpecSplit) and sp._local.shape == (4, 512 // size) and sp.shape == (4, 512)
        assert torch.equal(sp.to_broadcast()._local, c["x"])
        part = full.to_partial()
        assert isinstance(part.spec, CollectiveSpecPartial)
        assert torch.allclose(part.to_broadcast()._local.float(), c["x"].float(), atol=1e-2)

        # 2. column-parallel: outputs stay sharded; gathered they equal the full product
        col = ColumnParallelQLinear(c["qweight"], c["qzeros"], c["scales"], None, 4)
        y_local = col(c["x"])
        assert y_local.shape == (4, 128 // size)
        y = comm.all_gather(y_local, 1)
        assert torch.allclose(y.float(), ref, atol=2e-2, rtol=1e-2)

        # 3. row-parallel: x sliced on K, one all-reduce of the partial, bias counted once
        row = RowParallelQLinear(comm, c["qweight"], c["qzeros"], c["scales"], None, 4, bias=c["bias"])
        ks = 512 // size
        x_local = c["x"][:, ks * rank:ks * (rank + 1)].contiguous()
        z = row(x_local)
        assert torch.allclose(z.float(), ref + c["bias"].float(), atol=3e-2, rtol=1e-2)

        # 4. the MatrixMultiply rule on a CollectiveTensor x and a sharded quantized weight
        out = matrix_multiply(full, col.shard)
        assert isinstance(out.spec, CollectiveSpecSplit) and out.spec.axis == 1
        assert torch.allclose(out.to_broadcast()._local.float(), ref, atol=2e-2, rtol=1e-2)
        row_nb = RowParallelQLinear(comm, c["qweight"], c["qzeros"], c["scales"], None, 4)
        outp = matrix_multiply(full, row_nb.shard)
        assert isinstance(outp.spec, CollectiveSpecPartial)
        assert torch.allclose(outp.to_broadcast()._local.float(), ref, atol=3e-2, rtol=1e-2)

        # 5. row-parallel with act-order keeps the full scale table and slices g_idx
        ca = O.make_gptq_case(256, 64, 2, bits=4, act_order=True, seed=3)
        qw, qz, s, gi = shard_gptq_row(ca["qweight"], ca["qzeros"], ca["scales"], 4, rank, size, ca["g_idx"])
        assert s.shape == ca["scales"].shape and gi.shape == (256 // size,)
        wa = O.dequantize_packed(ca["qweight"], ca["g_idx"], ca["qzeros"], ca["scales"], 4)
        pa = ca["x"][:, 256 // size * rank:256 // size * (rank + 1)].float() @ O.dequantize_packed(qw, gi, qz, s, 4).float()
        assert torch.allclose(comm.all_reduce(pa), ca["x"].float() @ wa.float(), atol=1e-3)

        # 7. a checkpoint loaded through a sharding epilogue (examples/llama3_70b.py:298-310): the full shape is
        # checked first, then the epilogue's result is stored, a CollectiveTensor or a torch shard
        import tempfile
        from minit_b200 import checkpoint as C
        from minit_b200.module import Module

        class Net(Module):
            def __init__(self):
                super().__init__()
                self.w_col = self.register_buffer("w_col", (8, 6), "float16")
                self.w_row = self.register_buffer("w_row", (8, 6), "float16")
        full_w = {"w_col": torch.arange(48, dtype=torch.float16).reshape(8, 6), "w_row": -torch.arange(48, dtype=torch.float16).reshape(8, 6)}
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, f"net{rank}.safetensors")
            C.save_safetensors(path, full_w)

            def epilogue(key, value):
                ct = CollectiveTensor.from_broadcast(comm, value)
                return ct.to_split(0) if key == "w_col" else ct.to_split(1)._local       # a CollectiveTensor and a plain shard
            net = C.load_from_safetensors(Net(), [path], epilogue, device="cpu")
            assert isinstance(net.w_col, CollectiveTensor) and net.w_col.shape == (8, 6)
            assert torch.equal(net.w_col._local, full_w["w_col"][4 * rank:4 * rank + 4])
            assert torch.equal(net.w_row, full_w["w_row"][:, 3 * rank:3 * rank + 3])
            C.save_safetensors(path, {"w_col": torch.zeros(4, 6, dtype=torch.float16)})    # wrong full shape: refused before the epilogue
            with pytest.raises(ValueError):
                C.load_from_safetensors(Net(), [path], epilogue, device="cpu")

        # 6. shapes that do not split are refused
        with pytest.raises(ValueError):
            shard_gptq_column(c["qweight"][:, :24], c["qzeros"][:, :3], c["scales"][:, :24], 4, rank, size * 2 if size == 2 else 5)
        results[rank] = "ok"
    except BaseException as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(type(e), e, e.__traceback__))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_tensor_parallel_on_two_gloo_ranks():
    size = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(size, port, results), nprocs=size, join=True)
        for r in range(size):
            assert results.get(r) == "ok", f"rank {r}: {results.get(r)}"


def test_failed_rank_is_reported_not_hung():
    """A rank that raises before joining a collective is seen by the launcher as a failure
    (host-side fault injection; no GPU involved)."""
    def _bad(rank, size, port):
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import datetime
        dist.init_process_group("gloo", rank=rank, world_size=size, timeout=datetime.timedelta(seconds=10))
        if rank == 1:
            raise RuntimeError("injected failure on rank 1")
        t = torch.ones(1)
        dist.all_reduce(t)   # rank 0 must not wait forever for the dead rank

    with pytest.raises(Exception):
        mp.spawn(_bad, args=(2, _free_port()), nprocs=2, join=True)
