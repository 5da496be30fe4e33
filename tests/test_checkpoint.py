"""Checkpoint ingest (minit_b200/checkpoint.py) and the minit.* aliases, on CPU; the GPU part loads a sharded
act-order GPTQ model and runs it."""
import json
import os

import pytest
import torch

from oracle import qlinear_oracle as O


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def _tensors():
    g = torch.Generator().manual_seed(3)
    return {
        "layer.qweight": torch.randint(-2**31, 2**31 - 1, (16, 24), dtype=torch.int32, generator=g),
        "layer.scales": torch.randn(2, 24, generator=g).half(),
        "norm.weight": torch.randn(7, generator=g).bfloat16(),
        "count": torch.tensor(5, dtype=torch.int64),
        "mask": torch.tensor([True, False, True]),
        "bytes": torch.arange(-4, 4, dtype=torch.int8),
    }


def test_safetensors_roundtrip_and_format(M, tmp_path):
    from minit_b200 import checkpoint as C
    t = _tensors()
    p = str(tmp_path / "a.safetensors")
    C.save_safetensors(p, t, {"format": "pt"})
    got = dict(C.read_safetensors(p))
    assert list(got) == list(t)
    for k in t:
        assert got[k].dtype == t[k].dtype and torch.equal(got[k], t[k]), k
    st = pytest.importorskip("safetensors")
    from safetensors.torch import save_file
    with st.safe_open(p, framework="pt") as f:               # the library reads what we write
        for k in f.keys():
            assert torch.equal(f.get_tensor(k), t[k]), k
    q = str(tmp_path / "b.safetensors")
    save_file({k: v for k, v in t.items()}, q)               # and we read what the library writes
    got = dict(C.read_safetensors(q))
    for k in t:
        assert torch.equal(got[k], t[k]), k


def test_truncated_file_is_rejected(M, tmp_path):
    from minit_b200 import checkpoint as C
    p = str(tmp_path / "a.safetensors")
    C.save_safetensors(p, _tensors())
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-5])
    with pytest.raises(ValueError):
        dict(C.read_safetensors(p))


def _model(M, k, n, groups, bits):
    class Block(M.module.Module):
        def __init__(self):
            super().__init__()
            self.up = self.register_module("up", M.QLinear(k, n, groups, bits=bits))
            self.down = self.register_module("down", M.QLinearWithBias(n, k, n // 128, bits=bits))

        def forward(self, x):
            return self.down(self.up(x) * 0.05)
    return Block()


def _write_sharded(tmp_path, c_up, c_down):
    from minit_b200 import checkpoint as C
    a = {f"up.{k}": c_up[k] for k in ("qweight", "qzeros", "scales", "g_idx")}
    b = {f"down.{k}": c_down[k] for k in ("qweight", "qzeros", "scales", "g_idx", "bias")}
    C.save_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    C.save_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    index = {"metadata": {}, "weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a},
                                            **{k: "model-00002-of-00002.safetensors" for k in b}}}
    path = str(tmp_path / "model.safetensors.index.json")
    json.dump(index, open(path, "w"))
    return path


def test_index_loading_fills_buffers_and_checks_shapes(M, tmp_path):
    from minit_b200 import checkpoint as C
    c_up = O.make_gptq_case(256, 512, 1, bits=4, act_order=True, seed=1)
    c_down = O.make_gptq_case(512, 256, 1, bits=4, seed=2, bias=True)
    path = _write_sharded(tmp_path, c_up, c_down)
    model = _model(M, 256, 512, 2, 4)
    seen = []
    C.load_from_safetensors_index(model, path, epilogue=lambda k, v: (seen.append(k), v)[1], device="cpu")
    assert sorted(seen) == sorted([f"up.{k}" for k in ("qweight", "qzeros", "scales", "g_idx")] +
                                  [f"down.{k}" for k in ("qweight", "qzeros", "scales", "g_idx", "bias")])
    assert torch.equal(model.up.qweight, c_up["qweight"]) and torch.equal(model.down.bias, c_down["bias"])
    wrong = _model(M, 256, 384, 2, 4)                        # a model whose buffers do not fit the file
    with pytest.raises(ValueError):
        C.load_from_safetensors_index(wrong, path, device="cpu")


def test_minit_aliases(M):
    import sys
    from minit_b200 import compat
    had = "minit" in sys.modules
    assert compat.install() or had
    from minit.quantize.tensor import QuantizedTensor
    from minit.module.checkpoint import load_from_safetensors_index
    from minit.operator.linalg import MatrixMultiply
    assert QuantizedTensor is M.QuantizedTensor and MatrixMultiply is M.MatrixMultiply
    assert load_from_safetensors_index.__module__ == "minit_b200.checkpoint"


@pytest.mark.gpu
def test_sharded_act_order_model_loads_and_runs(M, tmp_path):
    from minit_b200 import checkpoint as C
    from tests.gpu_util import assert_close
    c_up = O.make_gptq_case(1024, 2048, 3, bits=4, act_order=True, seed=11)
    c_down = O.make_gptq_case(2048, 1024, 3, bits=4, act_order=True, seed=12, bias=True)
    path = _write_sharded(tmp_path, c_up, c_down)
    model = _model(M, 1024, 2048, 8, 4)
    C.load_from_safetensors_index(model, path, device="cuda:0", prepare=True)
    assert model.up._sorted not in (None, False) and model.down._sorted not in (None, False)
    x = c_up["x"].to("cuda:0")
    y = model(x)
    w1 = O.dequantize_packed(c_up["qweight"], c_up["g_idx"], c_up["qzeros"], c_up["scales"], 4)
    w2 = O.dequantize_packed(c_down["qweight"], c_down["g_idx"], c_down["qzeros"], c_down["scales"], 4)
    ref = O.qlinear(O.qlinear(c_up["x"], w1) * 0.05, w2, c_down["bias"])
    ok, err, bound = O.tolerance_ok(y, ref, 2e-2)                # two chained linears
    assert ok, f"err {err} > {bound}"
    assert_close(model.up(x[:1]), O.qlinear(c_up["x"][:1], w1), "first layer, M=1")
