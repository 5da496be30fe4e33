"""Tensor-parallel model code written against MiniT's Python surface, on two CPU ranks (gloo): ``CollectiveTensor`` as provided
by ``minit_b200.compat`` (placements, the gather-compute-broadcast rule of the functional layer, the column- / row-parallel
rules of ``matrix_multiply``).  Where the reference tree is present the model is examples/qwen1_5.py's own ``QWenLM`` at
toy sizes, sharded by the rule its collective server applies (examples/qwen1_5.py:311-321): q/k/v/gate/up split by
output features, o/down by input features."""
import importlib.util
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_root():
    for cand in (os.environ.get("MINIT_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "examples", "qwen1_5.py")):
            return cand
    return None


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, size, port, reference, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        from minit_b200 import compat
        from minit_b200.compat import tensor as T
        compat.install()
        T.set_device("cpu")
        import minit.functional as F
        from minit.collective.tensor import CollectiveTensor
        from minit.cuda.tensor import CUDATensor
        from minit.distributed.communicator import DistributedCommunicator
        from minit.distributed.group import initialize_world
        from minit_b200.collective.spec import CollectiveSpecBroadcast, CollectiveSpecPartial, CollectiveSpecSplit
        from minit_b200.distributed.torchdist import TorchDistTensor
        initialize_world(rank, size)
        comm = DistributedCommunicator(TorchDistTensor())
        g = torch.Generator().manual_seed(7)                       # the same numbers on every rank

        # 1. placements and the functional rule
        a = torch.randn((4, 6), generator=g)
        full = CollectiveTensor.from_broadcast(comm, CUDATensor.from_torch(a))
        sp = full.to_split(1)
        assert isinstance(sp.spec, CollectiveSpecSplit) and sp._local._shape == (4, 6 // size) and [d.item() for d in sp.shape] == [4, 6]
        assert np.array_equal(sp.numpy(), a.numpy()) and np.allclose(full.to_partial().numpy(), a.numpy(), atol=1e-6)
        assert isinstance(full.to_partial().spec, CollectiveSpecPartial)
        uni = CollectiveTensor.from_unique(comm, CUDATensor.from_torch(a + rank), 1)
        assert np.allclose(uni.numpy(), (a + 1).numpy())
        doubled = sp * 2 + 1                                          # any operator: gathered, computed whole, broadcast-placed
        assert isinstance(doubled, CollectiveTensor) and isinstance(doubled.spec, CollectiveSpecBroadcast)
        assert np.allclose(doubled.numpy(), (a * 2 + 1).numpy())
        assert sp.rearrange("a(bc)->abc", {"b": 2})._shape == (4, 2, 3) and (sp.shape[0] + 1).item() == 5
        assert F.tie([sp, full], axis=0)._shape == (8, 6) and len(sp.shape) == 2

        # 2. column- then row-parallel linears: the product of the first stays split, the second leaves a partial sum
        w1, w2 = torch.randn((8, 6), generator=g), torch.randn((5, 8), generator=g)
        x = torch.randn((2, 3, 6), generator=g)
        cw1 = CollectiveTensor.from_broadcast(comm, w1).to_split(0)   # torch locals, as a checkpoint epilogue produces them
        cw2 = CollectiveTensor.from_broadcast(comm, w2).to_split(1)
        cx = CollectiveTensor.from_broadcast(comm, CUDATensor.from_torch(x))
        h = F.matrix_multiply(cx, cw1)
        assert isinstance(h.spec, CollectiveSpecSplit) and h.spec.axis == 2 and h._local._shape == (2, 3, 8 // size)
        y = F.matrix_multiply(h, cw2)
        assert isinstance(y.spec, CollectiveSpecPartial) and y._shape == (2, 3, 5)
        assert np.allclose(y.numpy(), (x @ w1.t() @ w2.t()).numpy(), atol=1e-5)
        assert np.allclose(F.matrix_multiply(cx, CollectiveTensor.from_broadcast(comm, w1)).numpy(), (x @ w1.t()).numpy(), atol=1e-5)

        # 2b. the same pair with sharded GPTQ weights (CPU ranks have no kernel: the local product is the oracle's)
        from oracle import qlinear_oracle as O
        import minit_b200.collective.quantized as Q
        from minit_b200.collective import shard_gptq_column, shard_gptq_row

        def cpu_qmm(x, qweight, zeros, scales, groups, *, bits=8, bias=None, out=None, flags=0):
            return O.qlinear(x, O.dequantize_packed(qweight, groups, zeros, scales, bits), bias)
        Q.quantized_matrix_multiply = cpu_qmm
        c1 = O.make_gptq_case(256, 512, 6, bits=4, seed=3)
        c2 = O.make_gptq_case(512, 128, 6, bits=4, seed=4)
        q1 = Q.ShardedQuantized("column", *shard_gptq_column(c1["qweight"], c1["qzeros"], c1["scales"], 4, rank, size)[:3], None, 4)
        q2 = Q.ShardedQuantized("row", *shard_gptq_row(c2["qweight"], c2["qzeros"], c2["scales"], 4, rank, size)[:3], None, 4)
        xq = CollectiveTensor.from_broadcast(comm, CUDATensor.from_torch(c1["x"].reshape(2, 3, 256)))
        hq = F.matrix_multiply(xq, q1)
        assert isinstance(hq.spec, CollectiveSpecSplit) and hq.spec.axis == 2 and hq._local._shape == (2, 3, 512 // size)
        yq = F.matrix_multiply(hq * 0.05, q2)                        # the scaling gathers; the row-parallel rule slices again
        assert isinstance(yq.spec, CollectiveSpecPartial) and yq._shape == (2, 3, 128)
        w1q = O.dequantize_packed(c1["qweight"], None, c1["qzeros"], c1["scales"], 4)
        w2q = O.dequantize_packed(c2["qweight"], None, c2["qzeros"], c2["scales"], 4)
        refq = O.qlinear((O.qlinear(c1["x"], w1q).float() * 0.05).half(), w2q).reshape(2, 3, 128)
        ok, err, bound = O.tolerance_ok(yq.local().as_torch(), refq, 2e-2)
        assert ok, f"sharded quantized pair: {err} > {bound}"

        # 3. the reference's own tensor-parallel example model, sharded as its collective server shards it
        if reference is not None:
            examples = os.path.join(reference, "examples")
            sys.path.insert(0, examples)
            spec = importlib.util.spec_from_file_location("reference_example_qwen1_5", os.path.join(examples, "qwen1_5.py"))
            ex = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(ex)
            ex.default_dtype = "float32"
            weights = {}

            def build(shard):
                model = ex.QWenLM(50, 2, 32, 4, 1, 8, 64)
                for name, buf in list(model.named_buffers()):
                    shape = T.to_immediate_shape(buf.shape)
                    if name not in weights:
                        weights[name] = torch.randn(shape, generator=g) * 0.2 if len(shape) == 2 else 1 + 0.1 * torch.randn(shape, generator=g)
                    value = weights[name]
                    if shard:
                        value = CollectiveTensor.from_broadcast(comm, value)
                        if any(k in name for k in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "up_proj.weight", "gate_proj.weight")):
                            value = value.to_split(0)
                        elif "o_proj.weight" in name or "down_proj.weight" in name:
                            value = value.to_split(1)
                    model.update_buffer(name, value)
                return model

            ids = torch.tensor([[3, 7, 11, 2, 9]], dtype=torch.int32)
            plain = build(False)
            expect = plain.forward(CUDATensor.from_numpy(ids), F.constant(0, "int32"), plain.create_kv_caches()).numpy()
            model = build(True)
            model.model.freqs_cos = CollectiveTensor.from_broadcast(comm, model.model.freqs_cos)
            model.model.freqs_sin = CollectiveTensor.from_broadcast(comm, model.model.freqs_sin)
            caches = [(CollectiveTensor.from_broadcast(comm, k), CollectiveTensor.from_broadcast(comm, v)) for k, v in model.create_kv_caches()]
            out = model.forward(CollectiveTensor.from_broadcast(comm, CUDATensor.from_numpy(ids)),
                                CollectiveTensor.from_broadcast(comm, F.constant(0, "int32")), caches)
            assert isinstance(out, CollectiveTensor) and out._shape == (1, 5, 50)
            assert np.allclose(out.numpy(), expect, atol=1e-4), float(np.abs(out.numpy() - expect).max())
            last = out[0][out.shape[1] - 1]                           # what the server hands to the sampler
            assert np.allclose(last.numpy(), expect[0, 4], atol=1e-4)
        results[rank] = "ok"
    except Exception as e:                                            # report, do not hang the other rank
        import traceback
        results[rank] = traceback.format_exc()
        raise
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_model_code_on_two_gloo_ranks():
    size = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(size, _free_port(), _reference_root(), results), nprocs=size, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}, dict(results)
