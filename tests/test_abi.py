"""The C-ABI library loads without a GPU and exports every symbol include/minit_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "minit_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([a-z_0-9]+)\s*\(", text)
    return sorted({n for n in names if n.startswith(("mt_", "nccl_"))})


def test_header_symbols_are_exported_and_bound(lib_built):
    lib = ctypes.CDLL(lib_built)
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/minit_b200.h but not exported"
    from minit_b200 import _lib
    assert sorted(_lib.SYMBOLS) == names, "the ctypes table and the header disagree"


def test_host_only_entry_points(lib_built):
    from minit_b200 import _lib
    assert _lib.lib.mt_version() >= 100
    assert _lib.lib.mt_strerror(0) == b"ok"
    assert b"16-byte" in _lib.lib.mt_strerror(-2)
    assert _lib.lib.mt_workspace_bytes(1, 4096, 4096, 4) >= 16384
    assert _lib.lib.nccl_unique_id_size() == 128


def test_argument_validation_needs_no_gpu(lib_built):
    """Bad arguments are rejected on the host before any CUDA call."""
    from minit_b200 import _lib
    L = _lib.lib
    a = 1 << 20  # a fake, aligned, never dereferenced address
    # bits
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 1, 64, 64, 1, 3, 0, a, 1 << 20, 0) == -5
    # dtype
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 1, 64, 64, 1, 4, 7, a, 1 << 20, 0) == -4
    # n not a multiple of 8 / k not a multiple of 32 / groups do not divide k
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 1, 60, 64, 1, 4, 0, a, 1 << 20, 0) == -3
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 1, 64, 48, 1, 4, 0, a, 1 << 20, 0) == -3
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 1, 64, 64, 3, 4, 0, a, 1 << 20, 0) == -3
    # null and misaligned pointers
    assert L.mt_qgemm(None, None, a, None, a, a, None, a, 1, 64, 64, 1, 4, 0, a, 1 << 20, 0) == -1
    assert L.mt_qgemm(None, a + 2, a, None, a, a, None, a, 1, 64, 64, 1, 4, 0, a, 1 << 20, 0) == -2
    assert L.mt_dequant(None, a, None, a, a, None, 64, 64, 1, 4, 0) == -1
    assert L.mt_w8_perchannel_gemm(None, a, a, a, None, a, 1, 24, 64, 0, a, 1 << 20, 0) == -3
    # empty problems are a no-op
    assert L.mt_qgemm(None, a, a, None, a, a, None, a, 0, 64, 64, 1, 4, 0, a, 1 << 20, 0) == 0


def test_python_layer_refuses_cpu_tensors(lib_built):
    import torch
    import minit_b200 as M
    x = torch.zeros(1, 64, dtype=torch.float16)
    qw = torch.zeros(8, 64, dtype=torch.int32)
    qz = torch.zeros(1, 8, dtype=torch.int32)
    s = torch.ones(1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        M.quantized_matrix_multiply(x, qw, qz, s, None, bits=4)
    with pytest.raises(ValueError, match="shape mismatch"):
        M.quantized_matrix_multiply(x, qw, qz, s, None, bits=8)
