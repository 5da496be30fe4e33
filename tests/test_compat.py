"""The layer that lets code written against MiniT's Python surface run on this package (``minit_b200.compat``):
tensor types, functional operators, einops, modules, compiler helpers -- on the host device, so no GPU is needed.
Operators are checked against numpy / the oracle's restatements of the reference kernels; when the reference tree is
present (``MINIT_REFERENCE`` or ``../reference``) its single-process example scripts are imported UNCHANGED and a
small model built from their classes is compared with a plain torch implementation."""
import importlib.util
import math
import os
import shutil
import sys

import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_root():
    for cand in (os.environ.get("MINIT_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "examples", "mistral_7b.py")):
            return cand
    return None


@pytest.fixture(scope="module")
def minit():
    """``minit.*`` aliases installed, tensors on the host."""
    from minit_b200 import compat
    from minit_b200.compat import tensor
    had = "minit" in sys.modules
    assert compat.install() or had
    tensor.set_device("cpu")
    yield sys.modules["minit"]
    tensor.set_device(None)


def _t(array):
    from minit.cuda.tensor import CUDATensor
    return CUDATensor.from_numpy(np.asarray(array))


def test_aliases_cover_what_the_examples_import(minit):
    import minit.functional as F
    from minit.compiler.cxx import CXXUnit, import_symbol           # noqa: F401
    from minit.compiler.template import substitude
    from minit.core.cache import cached
    from minit.core.tensor import Tensor
    from minit.cuda.compiler import nvcc                            # noqa: F401
    from minit.cuda.kernel.utils import get_cuda_dtype
    from minit.cuda.tensor import CUDATensor
    from minit.functional.arith import constant
    from minit.functional.generate import fill, generate_sequence   # noqa: F401
    from minit.functional.linalg import batch_matrix_multiply, matrix_multiply, triangle_upper   # noqa: F401
    from minit.functional.special import rms_norm, rope, sigmoid, softmax   # noqa: F401
    from minit.module import Module
    from minit.module.checkpoint import load_from_safetensors, load_from_torch   # noqa: F401
    from minit.module.list import ModuleList
    from minit.quantize.tensor import QuantizedTensor               # noqa: F401
    import minit.cuda.dispatch                                      # noqa: F401
    import minit.quantize.dispatch                                  # noqa: F401
    import nvtx
    assert issubclass(CUDATensor, Tensor) and issubclass(ModuleList, Module)
    assert substitude("a ${X} b ${X}", {"X": "1"}) == "a 1 b 1" and get_cuda_dtype("float16") == "__half"
    assert constant(3, "int32").item() == 3 and F.einsum is not None
    calls = []

    @cached()
    def once(a):
        calls.append(a)
        return a * 2
    assert once(2) == 4 and once(2) == 4 and calls == [2]

    @nvtx.annotate("decorated")
    def f():
        return 7
    with nvtx.annotate("block"):
        assert f() == 7


def test_cuda_tensor_surface(minit):
    from minit.cuda.tensor import CUDATensor
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    x = CUDATensor.from_numpy(a)
    assert x.dtype == "float32" and x.device == "cuda" and [d.item() for d in x.shape] == [2, 3, 4]
    assert np.array_equal(x.numpy(), a) and x.size.item() == 24 and x.type() is CUDATensor
    assert isinstance(x.data_ptr, int) and x.data_ptr == x.memory._pointer and x.memory._size == 96
    y = CUDATensor.from_numpy(torch.tensor([[1, 2, 3]], dtype=torch.int32))     # the examples pass torch tensors here
    assert y.dtype == "int32" and y._shape == (1, 3)
    s = CUDATensor.from_item(2.5, "float16")
    assert s.item() == 2.5 and s._shape == () and s.numpy().dtype == np.float16
    z = CUDATensor.allocate((1, 0, 4, 8), "float16")                               # an empty KV cache
    assert z.numpy().shape == (1, 0, 4, 8)
    out = CUDATensor.allocate((3,), "int32")
    out._memory.reset()
    assert out.numpy().tolist() == [0, 0, 0]
    w = CUDATensor.wrap((6, 4), "float32", x.memory)                               # views share the memory
    w.as_torch()[0, 0] = 100.0
    assert x.numpy()[0, 0, 0] == 100.0
    with pytest.raises(AssertionError):
        CUDATensor.wrap((5, 4), "float32", x.memory)
    # indexing: whole slices of axis 0; bounds may be host scalars
    from minit.functional.arith import constant
    assert np.array_equal(x[1].numpy(), x.numpy()[1]) and np.array_equal(x[constant(0, "int32"):1].numpy(), x.numpy()[0:1])
    assert np.array_equal(x[1:].numpy(), x.numpy()[1:]) and x[:] is x


def test_shape_operators_are_views_or_copies_like_the_reference(minit):
    a = np.arange(2 * 3 * 4, dtype=np.int32).reshape(2, 3, 4)
    x = _t(a)
    assert np.array_equal(x.fold(0, 2).numpy(), a.reshape(6, 4)) and x.fold(1, 2) is x
    assert np.array_equal(x.expand(2, [2, 2]).numpy(), a.reshape(2, 3, 2, 2)) and x.expand(0, [2]) is x
    assert x.add_axis(1)._shape == (2, 1, 3, 4) and x.add_axis(1).remove_axis(1)._shape == (2, 3, 4)
    assert x.fold(0, 2).data_ptr == x.data_ptr and x.add_axis(0).data_ptr == x.data_ptr
    assert np.array_equal(x.add_axis(0, 5).numpy(), np.broadcast_to(a, (5, 2, 3, 4)))
    assert np.array_equal(x.transpose(2, 0).numpy(), a.transpose(2, 1, 0)) and x.transpose(1, 1) is x
    assert np.array_equal(x.repeat(1, 2).numpy(), np.tile(a, (1, 2, 1)))
    assert np.array_equal(x.repeat_interleaved(1, 2).numpy(), np.repeat(a, 2, axis=1))
    r = x.reinterpret("uint8")
    assert r._shape == (2, 3, 16) and np.array_equal(r.numpy(), a.view(np.uint8).reshape(2, 3, 16)) and r.data_ptr == x.data_ptr
    assert x.reinterpret("int64")._shape == (2, 3, 2)
    with pytest.raises(AssertionError):
        x.remove_axis(0)


def test_index_reduce_and_generators(minit):
    import minit.functional as F
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    x = _t(a)
    assert np.array_equal(x.slice(1, 3, 1).numpy(), a[:, 1:3])
    assert np.array_equal(x.index(_t(np.array([2, 0, 2], dtype=np.int32)), 1).numpy(), a[:, [2, 0, 2]])
    parts = x.split(2, [1, 3])
    assert [p._shape for p in parts] == [(2, 3, 1), (2, 3, 3)] and np.array_equal(F.tie(parts, axis=2).numpy(), a)
    v = _t(np.full((2, 1, 4), -1, dtype=np.float32))
    z = x.slice_set(1, 2, 1, v)
    assert np.array_equal(z.numpy()[:, 1], np.full((2, 4), -1)) and np.array_equal(x.numpy(), a)      # functional: x is untouched
    z = x.index_set(_t(np.array([0], dtype=np.int32)), 0, _t(np.zeros((1, 3, 4), dtype=np.float32)))
    assert z.numpy()[0].sum() == 0 and np.array_equal(z.numpy()[1], a[1])
    assert np.array_equal(x.sum(1).numpy(), a.sum(1, keepdims=True)) and np.array_equal(x.max(2).numpy(), a.max(2, keepdims=True))
    assert np.allclose(x.mean(0).numpy(), a.mean(0, keepdims=True))
    assert np.array_equal(F.generate_sequence(2, 4, 3, dtype="int32").numpy(), [2, 5, 8, 11])
    assert np.allclose(F.generate_sequence(0, 4, 0.25, dtype="float32").numpy(), [0, 0.25, 0.5, 0.75])
    assert np.array_equal(F.generate_interval(1, 7, 2, dtype="int32").numpy(), [1, 3, 5])
    f = F.fill(-math.inf, (x.shape[1], 2), "float16")
    assert f._shape == (3, 2) and f.dtype == "float16" and np.isneginf(f.numpy()).all()
    assert F.fill(F.constant(3, "int32"), (2,)).numpy().tolist() == [3, 3]


def test_arithmetic_rules(minit):
    import minit.functional as F
    h = _t(np.array([1.5, -2.0, 4.0], dtype=np.float16))
    assert (h + 1).dtype == "float16" and np.array_equal((h * 2).numpy(), [3.0, -4.0, 8.0])           # a number takes the tensor's dtype
    assert np.array_equal((1 - h).numpy(), np.float16([-0.5, 3.0, -3.0]))                              # reflected operators
    assert np.allclose((2.0 ** _t(np.array([0.0, 1.0, 3.0], dtype=np.float32))).numpy(), [1, 2, 8])
    i = _t(np.array([7, -7, 9], dtype=np.int32))
    assert (i / 2).numpy().tolist() == [3, -3, 4] and (i // 2).numpy().tolist() == [3, -4, 4] and (i % 4).numpy().tolist() == [3, 1, 1]
    assert (i > 0).dtype == "bool" and (i > 0).numpy().tolist() == [True, False, True]
    assert ((i > 0) & (i < 9)).numpy().tolist() == [True, False, False] and (i == 9).logical_not().numpy().tolist() == [True, True, False]
    assert F.where(i > 0, i, 0).numpy().tolist() == [7, 0, 9] and F.select_max(i, 8).numpy().tolist() == [8, 8, 9]
    assert h.cast("float32").dtype == "float32" and h.cast("float16") is h
    assert np.allclose(h.square().numpy(), [2.25, 4, 16]) and np.allclose(_t(np.float32([4, 9])).square_root().numpy(), [2, 3])
    assert np.allclose(_t(np.float32([0.0])).cosine().numpy(), [1]) and np.allclose(_t(np.float32([0.0])).exponential().numpy(), [1])
    # host scalars: dimensions and offsets stay on the host with their dtype
    a, b = F.constant(7, "int32"), F.constant(2, "int32")
    assert (a + b).item() == 9 and (a * 3).item() == 21 and (a // b).item() == 3 and (a / b).item() == 3 and (10 - a).item() == 3
    assert bool(a == 7) and not bool(a < b) and (a + b).dtype == "int32" and range(b).stop == 2
    assert (F.constant(1.0, "float32") / 4).item() == 0.25
    with pytest.raises(AssertionError):
        h + _t(np.array([1.0, 2.0, 3.0], dtype=np.float32))                                               # dtypes must agree


def test_special_functions_follow_the_oracle(minit):
    import minit.functional as F
    g = torch.Generator().manual_seed(3)
    x = torch.randn((2, 5, 4, 16), generator=g).half()
    w = (1 + 0.1 * torch.randn(16, generator=g)).half()
    out = F.rms_norm(_t(x), _t(w), 3, 1e-5).as_torch()
    ref = O.rms_norm(x, w, 1e-5)
    assert (out.float() - ref.float()).abs().max() <= 2e-3 * ref.float().abs().max()
    cos, sin = O.rope_tables(16, 32, 1e6)
    rot = F.rope(_t(x), _t(cos[3:8].contiguous()), _t(sin[3:8].contiguous())).as_torch()
    for b in range(2):
        assert torch.equal(rot[b], O.rope(x[b], cos, sin, 3))
    sm = F.softmax(_t(x), 1).as_torch()
    assert torch.equal(sm, torch.softmax(x.float(), 1).half())
    sg = F.sigmoid(_t(x)).as_torch()
    assert (sg.float() - O.sigmoid(x).float()).abs().max() <= 1e-3
    m = F.triangle_upper(F.fill(-math.inf, (4, 4), "float32"), diagonal=1).numpy()
    assert np.array_equal(np.isneginf(m), np.triu(np.ones((4, 4), bool), 1)) and (m[~np.isneginf(m)] == 0).all()
    t = F.triangle_lower(_t(np.ones((3, 3), dtype=np.float32)), 0).numpy()
    assert np.array_equal(t, np.tril(np.ones((3, 3)), -1))


def test_matrix_products(minit):
    import minit.functional as F
    g = np.random.default_rng(0)
    x, w = g.standard_normal((2, 3, 8), dtype=np.float32), g.standard_normal((5, 8), dtype=np.float32)
    out = F.matrix_multiply(_t(x), _t(w))                                # weights are [out, in]; leading axes fold
    assert out._shape == (2, 3, 5) and np.allclose(out.numpy(), x @ w.T, atol=1e-5)
    a, b = g.standard_normal((2, 4, 3, 8), dtype=np.float32), g.standard_normal((2, 4, 6, 8), dtype=np.float32)
    assert np.allclose(F.batch_matrix_multiply(_t(a), _t(b)).numpy(), a @ b.transpose(0, 1, 3, 2), atol=1e-5)


def test_einsum_and_rearrange(minit):
    import minit.functional as F
    g = np.random.default_rng(1)
    x = g.standard_normal((2, 3, 8), dtype=np.float32)
    q = _t(x).rearrange("bs(hd)->bshd", {"h": 2, "d": 4})
    assert np.array_equal(q.numpy(), x.reshape(2, 3, 2, 4))
    k = _t(x).rearrange("bs(hd)->bs(hr)d", {"h": 2, "d": 4, "r": 3})   # every head three times in a row
    assert np.array_equal(k.numpy(), np.repeat(x.reshape(2, 3, 2, 4), 3, axis=2))
    variables = {}
    flat = _t(np.arange(6, dtype=np.int32).reshape(2, 3)).rearrange("bs->(bs)", variables)
    assert flat._shape == (6,) and variables["b"].item() == 2 and variables["s"].item() == 3
    rows = _t(g.standard_normal((6, 5), dtype=np.float32))
    assert rows.rearrange("(bs)->bs", variables)._shape == (2, 3, 5)     # axes the equation does not name stay
    m = _t(np.arange(6, dtype=np.float32).reshape(2, 3)).rearrange("st->bnst", {"b": 2, "n": 4})
    assert m._shape == (2, 4, 2, 3) and np.array_equal(m.numpy()[1, 3], np.arange(6).reshape(2, 3))
    assert np.array_equal(_t(x).rearrange("...d->d...").numpy(), x.transpose(2, 0, 1))
    a, b = g.standard_normal((2, 3, 4, 5), dtype=np.float32), g.standard_normal((2, 6, 4, 5), dtype=np.float32)
    qk = F.einsum("bsnd,btnd->bnst", _t(a), _t(b))
    assert np.allclose(qk.numpy(), np.einsum("bsnd,btnd->bnst", a, b), atol=1e-5)
    o = F.einsum("bnst,btnd->bs(nd)", qk, _t(b))
    assert np.allclose(o.numpy(), np.einsum("bnst,btnd->bsnd", qk.numpy(), b).reshape(2, 3, 20), atol=1e-4)
    outer = F.einsum("a,b->ab", F.generate_sequence(0, 3, 1, dtype="float32"), F.generate_sequence(1, 2, 1, dtype="float32"))
    assert np.array_equal(outer.numpy(), np.outer([0, 1, 2], [1, 2]))
    with pytest.raises(AssertionError):
        _t(x).rearrange("bs(hd)->bshd", {"h": 3, "d": 4})


def test_modules_and_checkpoint_loader(minit, tmp_path):
    from minit.core.tensor import Tensor
    from minit.cuda.tensor import CUDATensor
    from minit.module import Module
    from minit.module.checkpoint import load_from_safetensors
    from minit.module.list import ModuleList
    import minit.functional as F
    from minit_b200.checkpoint import save_safetensors

    class Linear(Module):
        weight: Tensor

        def __init__(self, k, n):
            super().__init__()
            self.weight = self.register_buffer("weight", (n, k), "float32")

        def forward(self, x):
            return F.matrix_multiply(x, self.weight)

    class Stack(Module):
        layers: ModuleList[Linear]

        def __init__(self):
            super().__init__()
            self.layers = self.register_module("layers", ModuleList())
            for _ in range(2):
                self.layers.append(Linear(4, 4))

        def forward(self, x):
            for layer in self.layers:
                x = layer(x)
            return x

    model = Stack()
    assert [name for name, _ in model.named_buffers()] == ["layers.0.weight", "layers.1.weight"]
    spec = model.get_buffer("layers.1.weight")
    assert spec.device == "meta" and spec.dtype == "float32" and [d.item() for d in spec.shape] == [4, 4]
    w0, w1 = torch.randn(4, 4), torch.randn(4, 4)
    path = str(tmp_path / "model.safetensors")
    save_safetensors(path, {"layers.0.weight": w0, "layers.1.weight": w1})
    load_from_safetensors(model, [path], device="cpu")
    assert isinstance(model.layers[0].weight, CUDATensor) and len(model.layers) == 2
    x = torch.randn(3, 4)
    assert np.allclose(model(_t(x.numpy())).numpy(), (x @ w0.t() @ w1.t()).numpy(), atol=1e-5)
    with pytest.raises(ValueError):
        model.update_buffer("layers.0.weight", torch.zeros(4, 5))
    with pytest.raises(ValueError):
        model.update_buffer("layers.0.weight", torch.zeros(4, 4, dtype=torch.float16))


def test_chat_interfaces_drive_a_session(minit):
    from minit.chat.agent import Agent
    from minit.chat.sample import Top1Sampler
    from minit.chat.server import CacheKeyValueSession, Server
    from minit.chat.template import Template
    from minit.chat.tokenizer import Tokenizer

    class Echo(Server[CacheKeyValueSession]):
        """scores that make the sampler return the last input id + 1, and 0 (the end marker) after 3"""

        def create_session(self):
            return CacheKeyValueSession([])

        def decode(self, session, input_ids):
            session.offset += len(input_ids)
            scores = np.zeros(8, dtype=np.float32)
            scores[(input_ids[-1] + 1) if input_ids[-1] < 3 else 0] = 1.0
            return _t(scores)

    class Digits(Tokenizer):
        def tokenize(self, text):
            return [int(c) for c in text]

        def detokenize(self, ids):
            return "".join(str(i) for i in ids)

    class Plain(Template):
        def generate_header(self):
            return ""

        def generate_prompt(self, prompt):
            return prompt

        def generate(self, user):
            return user, "0"

        def eos(self):
            return "0"

    server = Echo()
    agent = Agent(server, Digits(), Plain(), Top1Sampler())
    session = agent.create_session(None)
    assert session.interact("1") == "23"                               # 1 -> 2 -> 3 -> end marker


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_runtime_compiled_unit_and_imported_symbol(minit, tmp_path, monkeypatch):
    import ctypes
    from minit.compiler.cxx import CXXUnit, import_symbol
    from minit.cuda.compiler import nvcc
    monkeypatch.setenv("MINIT_B200_CACHE", str(tmp_path))
    unit = CXXUnit(source='extern "C" int scaled_sum(int a, int b) { return FACTOR * (a + b); }\n', defines=["FACTOR=3"])
    library = nvcc.compile(unit)

    @import_symbol(library, "scaled_sum")
    def scaled_sum(a: ctypes.c_int, b: ctypes.c_int) -> ctypes.c_int:
        ...
    assert scaled_sum(2, 5) == 21
    assert len(os.listdir(tmp_path)) == 1
    nvcc.compile(unit)                                                   # second request: served from the cache directory
    assert len(os.listdir(tmp_path)) == 1


# ---------------------------------------------------------------------------------------------------------------------
# the reference's own example scripts, imported unchanged (only where the reference tree is present)
# ---------------------------------------------------------------------------------------------------------------------
def _import_example(root, name):
    examples = os.path.join(root, "examples")
    if examples not in sys.path:
        sys.path.insert(0, examples)                                     # mistral_7b.py imports its neighbour agent.py
    spec = importlib.util.spec_from_file_location(f"reference_example_{name}", os.path.join(examples, f"{name}.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.skipif(_reference_root() is None, reason="reference tree not present")
def test_example_scripts_import_unchanged(minit):
    root = _reference_root()
    mistral = _import_example(root, "mistral_7b")
    qwen = _import_example(root, "qwen1_5_int8")
    qwen_tp = _import_example(root, "qwen1_5")                           # the tensor-parallel script: chat + collective + nccl modules
    from minit.module import Module
    assert issubclass(mistral.LlaMa2, Module) and issubclass(qwen.QLinearWithBias, Module) and issubclass(qwen_tp.Attention, Module)
    # the int8 example's own ``unpack`` (reinterpret, expand, add_axis, transpose, remove_axis, fold) agrees with the oracle
    c = O.make_gptq_case(64, 32, 1, bits=8, group_size=32, seed=4)
    assert np.array_equal(qwen.unpack(_t(c["qweight"].numpy()), 0).numpy(), O.unpack_rows(c["qweight"].numpy(), 8))
    assert np.array_equal(qwen.unpack(_t(c["qzeros"].numpy()), 1).numpy(), O.unpack_cols(c["qzeros"].numpy(), 8))
    lin = qwen.QLinear(64, 32, 2)
    for name in ("qweight", "qzeros", "scales", "g_idx"):
        lin.update_buffer(name, c[name])
    qt = lin.weight                                                       # QuantizedTensor(unpack(qweight), g_idx, unpack(qzeros), scales)
    assert tuple(qt.shape) == (64, 32) and qt._data.dtype == torch.uint8 and qt._zero.shape == (2, 32)
    assert np.array_equal(qt._data.numpy(), c["q"]) and np.array_equal(qt._zero.numpy(), c["z"])


@pytest.mark.skipif(_reference_root() is None, reason="reference tree not present")
def test_example_model_runs_and_matches_plain_torch(minit):
    """examples/mistral_7b.py's LlaMa2 at toy sizes in fp32: prefill of five tokens, then one cached decode step."""
    import minit.functional as F
    from minit.cuda.tensor import CUDATensor
    from minit_b200.compat.tensor import to_immediate_shape
    ex = _import_example(_reference_root(), "mistral_7b")
    ex.default_dtype = "float32"
    E, L, NQ, NG, D, I = 50, 2, 4, 2, 8, 64
    model = ex.LlaMa2(E, L, NQ * D, NQ, NG, D, I)
    g = torch.Generator().manual_seed(0)
    weights = {}
    for name, buf in list(model.named_buffers()):
        shape = to_immediate_shape(buf.shape)
        w = torch.randn(shape, generator=g) * 0.2 if len(shape) == 2 else 1 + 0.1 * torch.randn(shape, generator=g)
        weights[name] = w
        model.update_buffer(name, w)
    ids = torch.tensor([[3, 7, 11, 2, 9]], dtype=torch.int32)
    nxt = torch.tensor([[5]], dtype=torch.int32)
    caches = model.create_kv_caches()
    out = model.forward(CUDATensor.from_numpy(ids), F.constant(0, "int32"), caches)
    out2 = model.forward(CUDATensor.from_numpy(nxt), F.constant(5, "int32"), caches)
    assert out._shape == (1, 5, E) and out2._shape == (1, 1, E) and caches[0][0]._shape == (1, 6, NQ, D)

    def plain(tokens):
        s = tokens.shape[1]
        x = weights["tok_embeddings.weight"][tokens.long()]
        freqs = (1 / 1e6) ** (torch.arange(0, D // 2, dtype=torch.float32) * (2 / D))
        ang = torch.arange(s, dtype=torch.float32)[:, None] * freqs[None]
        cos, sin = ang.cos().view(1, s, 1, -1), ang.sin().view(1, s, 1, -1)

        def rot(t):
            p = t.reshape(1, s, -1, D // 2, 2)
            re, im = p[..., 0], p[..., 1]
            return torch.stack((re * cos - im * sin, im * cos + re * sin), -1).reshape(t.shape)

        def norm(t, w):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * w

        for layer in range(L):
            p = f"layers.{layer}."
            h = norm(x, weights[p + "attention_norm.weight"])
            q = rot((h @ weights[p + "attention.wq.weight"].t()).view(1, s, NQ, D))
            k = rot((h @ weights[p + "attention.wk.weight"].t()).view(1, s, NQ // NG, D).repeat_interleave(NG, dim=2))
            v = (h @ weights[p + "attention.wv.weight"].t()).view(1, s, NQ // NG, D).repeat_interleave(NG, dim=2)
            qk = torch.einsum("bsnd,btnd->bnst", q, k) / math.sqrt(D) + torch.triu(torch.full((s, s), -math.inf), 1)
            o = torch.einsum("bnst,btnd->bsnd", torch.softmax(qk, -1), v).reshape(1, s, NQ * D)
            x = x + o @ weights[p + "attention.wo.weight"].t()
            h = norm(x, weights[p + "ffn_norm.weight"])
            gate, up = h @ weights[p + "feed_forward.w1.weight"].t(), h @ weights[p + "feed_forward.w3.weight"].t()
            x = x + (gate * torch.sigmoid(gate) * up) @ weights[p + "feed_forward.w2.weight"].t()
        return norm(x, weights["norm.weight"]) @ weights["output.weight"].t()

    assert (out.as_torch() - plain(ids)).abs().max() < 1e-4
    assert (out2.as_torch() - plain(torch.cat([ids, nxt], 1))[:, -1:]).abs().max() < 1e-4


@pytest.mark.skipif(_reference_root() is None, reason="reference tree not present")
def test_tensor_parallel_example_model_runs_single_process(minit):
    """examples/qwen1_5.py's QWenLM (biased qkv linears, one KV group) at toy sizes: a cached decode step gives the scores
    of recomputing the whole sequence."""
    import minit.functional as F
    from minit.cuda.tensor import CUDATensor
    from minit_b200.compat.tensor import to_immediate_shape, torch_dtype
    ex = _import_example(_reference_root(), "qwen1_5")
    ex.default_dtype = "float32"
    model = ex.QWenLM(50, 2, 32, 4, 1, 8, 64)
    g = torch.Generator().manual_seed(1)
    for name, buf in list(model.named_buffers()):
        shape = to_immediate_shape(buf.shape)
        w = torch.randn(shape, generator=g) * 0.2 if len(shape) == 2 else 1 + 0.1 * torch.randn(shape, generator=g)
        model.update_buffer(name, w.to(torch_dtype(buf.dtype)))
    ids = torch.tensor([[3, 7, 11, 2, 9, 4]], dtype=torch.int32)
    full = model.forward(CUDATensor.from_numpy(ids), F.constant(0, "int32"), model.create_kv_caches())
    caches = model.create_kv_caches()
    model.forward(CUDATensor.from_numpy(ids[:, :5].contiguous()), F.constant(0, "int32"), caches)
    step = model.forward(CUDATensor.from_numpy(ids[:, 5:].contiguous()), F.constant(5, "int32"), caches)
    assert full._shape == (1, 6, 50) and step._shape == (1, 1, 50) and np.isfinite(full.numpy()).all()
    assert np.allclose(step.numpy()[0, 0], full.numpy()[0, 5], atol=1e-4)


@pytest.mark.skipif(_reference_root() is None or shutil.which("nvcc") is None, reason="needs the reference tree and nvcc")
def test_int8_example_builds_its_own_kernel_through_the_compiler_helpers(minit, tmp_path, monkeypatch):
    """examples/qwen1_5_int8.py:53-241 fills its CUDA source template, compiles it (``nvcc.compile(CXXUnit(...))``) and binds the
    entry point (``import_symbol``): all three helpers come from this package here; the build targets sm_100a."""
    import ctypes
    monkeypatch.setenv("MINIT_B200_CACHE", str(tmp_path))
    qwen = _import_example(_reference_root(), "qwen1_5_int8")
    entrance = qwen.generate_quantized_matrix_multiply("qmm_compat_test", "float16", "float16")
    assert entrance.argtypes == [ctypes.c_void_p] * 7 + [ctypes.c_int] * 4 and entrance.restype is None
    assert qwen.generate_quantized_matrix_multiply("qmm_compat_test", "float16", "float16") is entrance     # ``cached``


def test_register_dispatch_by_annotations(minit):
    """the reference's registration form (minit/core/dispatch.py:52-58): operator and operand classes from the annotations"""
    from dataclasses import dataclass
    from typing import Literal, Union
    from minit.core.dispatch import dispatch, register_dispatch
    from minit.core.operator import Operator
    from minit.core.tensor import Tensor
    from minit.cuda.tensor import CUDATensor
    from minit_b200.compat.tensor import ScalarTensor

    @dataclass
    class Scale(Operator):
        factor: float

    @dataclass
    class Negate(Operator):
        ...

    @register_dispatch()
    def scale_device(op: Scale, x: CUDATensor):
        return (x * op.factor,)

    @register_dispatch()
    def scale_host(op: Scale, x: ScalarTensor):
        return (ScalarTensor(x.value() * op.factor, (), x.dtype),)

    @register_dispatch(priority=1, predicate=lambda *types: len(types) == 2)       # the predicate sees the operand TYPES
    def scale_pair(op: Scale, *xs: Union[CUDATensor, ScalarTensor]):
        assert all(isinstance(t, type) for t in (type(x) for x in xs))
        return tuple(dispatch(op, x)[0] for x in xs)

    @register_dispatch()
    def any_unary(op: Union[Negate], x: Tensor):
        return (0 - x,)

    x = _t(np.float32([1, 2]))
    (y,) = dispatch(Scale(3.0), x)
    assert y.numpy().tolist() == [3, 6]
    (h,) = dispatch(Scale(2.0), ScalarTensor(4.0, (), "float32"))
    assert h.item() == 8.0
    a, b = dispatch(Scale(2.0), x, ScalarTensor(1.0, (), "float32"))                   # two operands: the higher-priority rule
    assert a.numpy().tolist() == [2, 4] and b.item() == 2.0
    assert dispatch(Negate(), x)[0].numpy().tolist() == [-1, -2]
    with pytest.raises(TypeError):
        dispatch(Scale(1.0), "text")
    with pytest.raises(TypeError):                                                      # parametrised patterns are refused
        @register_dispatch()
        def bad(op: Scale, x: Literal["cuda"]):
            return (x,)
    with pytest.raises(TypeError):
        @register_dispatch()
        def unannotated(op: Scale, x):
            return (x,)


def test_eager_stand_ins_for_the_tracer(minit, tmp_path):
    import minit.functional as F
    import minit.trace.dispatch                                         # noqa: F401  (imported by the scripts for its side effect)
    from minit.graph import dump_graphviz
    from minit.trace.executor import TraceGraphExecutor
    from minit.trace.function import trace_function

    def forward(x, offset, *rest):
        return (x * 2 + offset, *rest)

    x = _t(np.float32([1, 2, 3]))
    graph = trace_function(forward, (x, F.constant(1, "float32"), x))
    out, passed = TraceGraphExecutor(graph).execute(x, F.constant(1, "float32"), x)
    assert out.numpy().tolist() == [3, 5, 7] and passed is x
    dump_graphviz(graph).save(str(tmp_path / "graph.dot"))
    text = open(tmp_path / "graph.dot").read()
    assert text.startswith("digraph") and "forward (eager)" in text and "float32[3]" in text
    assert TraceGraphExecutor(trace_function(lambda: None, ())).execute() == ()


@pytest.mark.skipif(_reference_root() is None, reason="reference tree not present")
def test_traced_example_imports_and_its_model_runs_through_the_executor(minit):
    """examples/llama3.py (it wraps the forward pass in trace_function / TraceGraphExecutor, examples/llama3.py:360-367)"""
    import minit.functional as F
    from minit.cuda.tensor import CUDATensor
    from minit.trace.executor import TraceGraphExecutor
    from minit.trace.function import trace_function
    from minit_b200.compat.tensor import to_immediate_shape, torch_dtype
    ex = _import_example(_reference_root(), "llama3")
    ex.default_dtype = "float32"
    model = ex.Llama3LM(50, 2, 32, 4, 2, 8, 64)
    g = torch.Generator().manual_seed(2)
    for name, buf in list(model.named_buffers()):
        shape = to_immediate_shape(buf.shape)
        w = torch.randn(shape, generator=g) * 0.2 if len(shape) == 2 else 1 + 0.1 * torch.randn(shape, generator=g)
        model.update_buffer(name, w.to(torch_dtype(buf.dtype)))

    def model_forward(input, offset, *flat):
        caches = [(flat[2 * i], flat[2 * i + 1]) for i in range(len(flat) // 2)]
        probs = model.forward(input, offset, caches)
        return (probs, *[t for pair in caches for t in pair])

    def flat(caches):
        return [t for pair in caches for t in pair]

    ids = torch.tensor([[3, 7, 11, 2, 9, 4]], dtype=torch.int32)
    full_in = CUDATensor.from_numpy(ids)
    executor = TraceGraphExecutor(trace_function(model_forward, (full_in, F.constant(0, "int32"), *flat(model.create_kv_caches()))))
    full, *_ = executor.execute(full_in, F.constant(0, "int32"), *flat(model.create_kv_caches()))
    _, *kv = executor.execute(CUDATensor.from_numpy(ids[:, :5].contiguous()), F.constant(0, "int32"), *flat(model.create_kv_caches()))
    step, *_ = executor.execute(CUDATensor.from_numpy(ids[:, 5:].contiguous()), F.constant(5, "int32"), *kv)
    assert full._shape == (1, 6, 50) and step._shape == (1, 1, 50)
    assert np.allclose(step.numpy()[0, 0], full.numpy()[0, 5], atol=1e-4)
