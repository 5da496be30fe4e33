"""The reference's run-time C++/CUDA compilation helpers, for scripts that carry their own kernel source:
``CXXUnit`` / ``import_symbol`` (minit/compiler/cxx.py:18-59), ``substitude`` (minit/compiler/template.py:4-7),
``nvcc.compile`` (minit/cuda/compiler.py:9-28), ``get_cuda_dtype`` (minit/cuda/kernel/utils.py:1-17) and ``cached``
(minit/core/cache.py:5-17).  ``nvcc.compile`` builds for sm_100a (the reference asks for compute_70 PTX) into a
per-source directory of the user's cache and loads the library with ctypes."""
from __future__ import annotations

import ctypes
import functools
import hashlib
import inspect
import os
import shutil
import subprocess
from dataclasses import dataclass, field
from typing import Dict, List


def cached():
    def decorator(function):
        memo: Dict[tuple, object] = {}

        @functools.wraps(function)
        def decorated(*args):
            if args not in memo:
                memo[args] = function(*args)
            return memo[args]
        return decorated
    return decorator


def substitude(source: str, args: Dict[str, str]) -> str:
    for key, value in args.items():
        source = source.replace("${" + key + "}", value)
    return source


@dataclass
class CXXUnit:
    source: str
    includes: List[str] = field(default_factory=list)
    libraries: List[str] = field(default_factory=list)
    defines: List[str] = field(default_factory=list)


def import_symbol(cdll: ctypes.CDLL, name: str):
    """Decorator: the annotations of the decorated stub become the ctypes signature of ``cdll.<name>``, which is
    returned in the stub's place."""
    def decorator(function):
        signature = inspect.signature(function)
        symbol = getattr(cdll, name)
        symbol.argtypes = [parameter.annotation for parameter in signature.parameters.values()]
        symbol.restype = None if signature.return_annotation is signature.empty else signature.return_annotation
        return symbol
    return decorator


class CXXCompiler:
    def compile(self, unit: CXXUnit) -> ctypes.CDLL:
        raise NotImplementedError()


def _cache_root() -> str:
    return os.environ.get("MINIT_B200_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "minit_b200", "compiled")


class NVCC(CXXCompiler):
    arch = ["-gencode", "arch=compute_100a,code=sm_100a"]

    def compile(self, unit: CXXUnit) -> ctypes.CDLL:
        exe = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        command = [exe]
        for include in unit.includes:
            command += ["-I", include]
        for library in unit.libraries:
            command += ["-l", library]
        for define in unit.defines:
            command += ["-D", define]
        command += ["-shared", "--compiler-options", "-fPIC", *self.arch, "main.cu", "-o", "library.so"]
        key = hashlib.sha256((repr(command) + unit.source).encode()).hexdigest()[:16]
        directory = os.path.join(_cache_root(), key)
        library = os.path.join(directory, "library.so")
        if not os.path.exists(os.path.join(directory, ".done")):
            os.makedirs(directory, exist_ok=True)
            with open(os.path.join(directory, "main.cu"), "w") as f:
                f.write(unit.source)
            subprocess.check_call(command, cwd=directory)
            open(os.path.join(directory, ".done"), "w").close()
        return ctypes.CDLL(library)


nvcc = NVCC()

CUDA_DTYPE_MAPPING = {
    "bfloat16": "__nv_bfloat16", "float16": "__half", "float32": "float", "float64": "double",
    "int8": "std::int8_t", "int16": "std::int16_t", "int32": "std::int32_t", "int64": "std::int64_t",
    "uint8": "std::uint8_t", "uint16": "std::uint16_t", "uint32": "std::uint32_t", "uint64": "std::uint64_t",
}


def get_cuda_dtype(name: str) -> str:
    return CUDA_DTYPE_MAPPING[name]
