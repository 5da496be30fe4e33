"""Optional aliases under the reference's package name: ``minit_b200.compat.install()`` registers the
modules of this package that mirror MiniT's quantized-linear path as ``minit.*`` in ``sys.modules``
(only when no real ``minit`` is importable), so code written as ``from minit.quantize.tensor import
QuantizedTensor`` or ``from minit.module.checkpoint import load_from_safetensors_index`` finds them.
Only this path is covered: the rest of MiniT (tensor runtime, attention, graph layers) is not part of
this package and stays unavailable."""
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
    "minit.functional": "minit_b200.functional",
    "minit.functional.linalg": "minit_b200.functional.linalg",
    "minit.core.dispatch": "minit_b200.core.dispatch",
    "minit.core.operator": "minit_b200.core.operator",
    "minit.module": "minit_b200.module",
    "minit.module.checkpoint": "minit_b200.checkpoint",
    "minit.distributed": "minit_b200.distributed",
    "minit.distributed.group": "minit_b200.distributed.group",
    "minit.distributed.communicator": "minit_b200.distributed.communicator",
    "minit.nccl": "minit_b200.nccl",
    "minit.collective": "minit_b200.collective",
}


def install(force: bool = False) -> bool:
    """Register the aliases.  Returns False (and does nothing) when a real ``minit`` package is importable
    and ``force`` is not set."""
    if not force and "minit" not in sys.modules and importlib.util.find_spec("minit") is not None:
        return False
    root = sys.modules.get("minit")
    if root is None or force:
        root = types.ModuleType("minit")
        root.__path__ = []          # a package: submodules are resolved through sys.modules
        root.__doc__ = "aliases of minit_b200 (quantized-linear path only)"
        sys.modules["minit"] = root
    core = types.ModuleType("minit.core")
    core.__path__ = []
    sys.modules.setdefault("minit.core", core)
    setattr(root, "core", sys.modules["minit.core"])
    for alias, target in _ALIASES.items():
        mod = importlib.import_module(target)
        sys.modules[alias] = mod
        parent, _, leaf = alias.rpartition(".")
        setattr(sys.modules[parent], leaf, mod)
    return True
