"""Aliases under the reference's package name, for code written against MiniT.

``minit_b200.compat.install()`` registers modules of this package as ``minit.*`` in ``sys.modules`` (only when no
real ``minit`` is importable, unless forced), so that

* ``from minit.quantize.tensor import QuantizedTensor``, ``from minit.operator.linalg import MatrixMultiply``,
  ``from minit.module.checkpoint import load_from_safetensors_index`` and the distributed / collective / nccl
  modules resolve to this package's implementations of the quantized-linear path, and
* example scripts of the reference (examples/mistral_7b.py, examples/qwen1_5_int8.py, examples/qwen1_5.py,
  examples/llama3.py and the helper examples/agent.py) import unchanged: the tensor types (``minit.core.tensor``, ``minit.cuda.tensor``), the
  functional layer (``minit.functional`` and its submodules), ``minit.module`` / ``minit.module.list``, the
  run-time compiler helpers (``minit.compiler.cxx``, ``minit.compiler.template``, ``minit.cuda.compiler``,
  ``minit.cuda.kernel.utils``, ``minit.core.cache``), the interface classes of ``minit.chat`` and a stand-in for
  ``nvtx`` when that package is absent.
  These sit on torch storage and are plumbing around the hot path, which a model reaches through
  ``F.matrix_multiply(x, QuantizedTensor)`` or this package's ``QLinear``.

The graph tracer is NOT rebuilt: ``minit.trace.function.trace_function`` / ``minit.trace.executor.TraceGraphExecutor``
/ ``minit.graph.dump_graphviz`` are eager stand-ins (``compat/trace.py``: the function is kept and called).  Not
provided at all: lazy tensors and traced control flow (``minit.lazy``, for_loop / while_loop / if_block) and the
remote controller (``minit.remote``, ``minit.nccl.library.launch_server``) -- examples/llama3_70b.py needs those and
does not import."""
from __future__ import annotations

import importlib
import importlib.util
import sys
import types

_ALIASES = {
    "minit.quantize": "minit_b200.quantize",
    "minit.quantize.tensor": "minit_b200.quantize.tensor",
    "minit.quantize.operator": "minit_b200.quantize.operator",
    "minit.quantize.functional": "minit_b200.quantize.functional",
    "minit.operator": "minit_b200.operator",
    "minit.operator.linalg": "minit_b200.operator.linalg",
    "minit.core.dispatch": "minit_b200.core.dispatch",
    "minit.core.operator": "minit_b200.core.operator",
    "minit.core.tensor": "minit_b200.compat.tensor",
    "minit.core.scalar": "minit_b200.compat.tensor",
    "minit.core.meta": "minit_b200.compat.tensor",
    "minit.core.shape": "minit_b200.compat.tensor",
    "minit.core.dtype": "minit_b200.compat.tensor",
    "minit.core.cache": "minit_b200.compat.compiler",
    "minit.cuda.tensor": "minit_b200.compat.tensor",
    "minit.cuda.compiler": "minit_b200.compat.compiler",
    "minit.cuda.kernel.utils": "minit_b200.compat.compiler",
    "minit.compiler.cxx": "minit_b200.compat.compiler",
    "minit.compiler.template": "minit_b200.compat.compiler",
    "minit.functional": "minit_b200.compat.functional",
    "minit.functional.arith": "minit_b200.compat.functional.arith",
    "minit.functional.einops": "minit_b200.compat.functional.einops",
    "minit.functional.generate": "minit_b200.compat.functional.generate",
    "minit.functional.index": "minit_b200.compat.functional.index",
    "minit.functional.linalg": "minit_b200.compat.functional.linalg",
    "minit.functional.reduce": "minit_b200.compat.functional.reduce",
    "minit.functional.shape": "minit_b200.compat.functional.shape",
    "minit.functional.special": "minit_b200.compat.functional.special",
    "minit.module": "minit_b200.compat.module",
    "minit.module.module": "minit_b200.compat.module",
    "minit.module.list": "minit_b200.compat.module",
    "minit.module.checkpoint": "minit_b200.checkpoint",
    "minit.distributed": "minit_b200.distributed",
    "minit.distributed.group": "minit_b200.distributed.group",
    "minit.distributed.communicator": "minit_b200.distributed.communicator",
    "minit.distributed.operator": "minit_b200.distributed.operator",
    "minit.nccl": "minit_b200.nccl",
    "minit.nccl.tensor": "minit_b200.nccl.tensor",
    "minit.nccl.dispatch": "minit_b200.nccl.dispatch",
    "minit.nccl.library": "minit_b200.nccl.library",
    "minit.collective": "minit_b200.collective",
    "minit.collective.tensor": "minit_b200.compat.collective",
    "minit.collective.dispatch": "minit_b200.collective.dispatch",
    "minit.collective.spec": "minit_b200.collective.spec",
    "minit.trace.function": "minit_b200.compat.trace",
    "minit.trace.executor": "minit_b200.compat.trace",
    "minit.graph": "minit_b200.compat.trace",
    "minit.chat.server": "minit_b200.compat.chat",
    "minit.chat.sample": "minit_b200.compat.chat",
    "minit.chat.template": "minit_b200.compat.chat",
    "minit.chat.tokenizer": "minit_b200.compat.chat",
    "minit.chat.agent": "minit_b200.compat.chat",
}

# packages that exist only as containers, and modules the reference imports for their side effect (registering
# dispatch rules): the rules of this package are registered when its own modules load
_CONTAINERS = ("minit.core", "minit.cuda", "minit.cuda.kernel", "minit.compiler", "minit.chat", "minit.trace")
_SIDE_EFFECT_ONLY = ("minit.cuda.dispatch", "minit.quantize.dispatch", "minit.trace.dispatch")


class _Annotate:
    """``nvtx.annotate``: usable as a decorator and as a context manager; does nothing."""

    def __init__(self, *args, **kwargs) -> None:
        pass

    def __call__(self, function):
        return function

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> bool:
        return False


def _install_nvtx() -> None:
    if "nvtx" in sys.modules or importlib.util.find_spec("nvtx") is not None:
        return
    stub = types.ModuleType("nvtx")
    stub.__doc__ = "stand-in installed by minit_b200.compat: range annotations are dropped"
    stub.annotate = _Annotate
    stub.push_range = lambda *args, **kwargs: None
    stub.pop_range = lambda *args, **kwargs: None
    stub.mark = lambda *args, **kwargs: None
    sys.modules["nvtx"] = stub


def _container(name: str) -> types.ModuleType:
    module = sys.modules.get(name)
    if module is None:
        module = types.ModuleType(name)
        module.__path__ = []            # a package: submodules are resolved through sys.modules
        sys.modules[name] = module
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(_container(parent), leaf, module)
    return module


def install(force: bool = False) -> bool:
    """Register the aliases.  Returns False (and does nothing) when a real ``minit`` package is importable
    and ``force`` is not set."""
    if not force and "minit" not in sys.modules and importlib.util.find_spec("minit") is not None:
        return False
    if force or "minit" not in sys.modules:
        root = types.ModuleType("minit")
        root.__path__ = []
        root.__doc__ = "aliases of minit_b200 (quantized-linear path and the layer the single-process examples import)"
        sys.modules["minit"] = root
    for name in _CONTAINERS:
        _container(name)
    for alias, target in _ALIASES.items():
        module = importlib.import_module(target)
        sys.modules[alias] = module
        parent, _, leaf = alias.rpartition(".")
        setattr(_container(parent), leaf, module)
    for name in _SIDE_EFFECT_ONLY:
        if name not in sys.modules:
            module = types.ModuleType(name)
            module.__doc__ = "imported by the reference for its side effect; nothing to register here"
            sys.modules[name] = module
            parent, _, leaf = name.rpartition(".")
            setattr(_container(parent), leaf, module)
    _install_nvtx()
    return True
