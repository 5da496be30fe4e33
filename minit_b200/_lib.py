"""ctypes binding of libminit_b200.so -- the only route from Python to the kernels.

There is no fallback: if the library has not been built the import of this module raises,
and every call checks the returned status and raises on failure.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libminit_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python minit_b200/csrc/build.py` (needs nvcc). "
        "minit_b200 has no CPU or PyTorch fallback for its kernels.")

lib = ctypes.CDLL(LIB_PATH)

MT_F16, MT_BF16 = 0, 1
FLAG_FORCE_SMALL, FLAG_FORCE_TC, FLAG_PDL, FLAG_FORCE_VEC, FLAG_FORCE_UMMA, FLAG_AR_SHORT_WAIT, FLAG_FORCE_MID = 1, 2, 4, 16, 32, 64, 128
FLAG_TC_TMEM_A, FLAG_TC_SMEM_A, FLAG_AR_TWO_SHOT, FLAG_AR_ONE_SHOT = 256, 512, 1024, 2048
ERR_PEER_TIMEOUT = -12
ERR_UNSUPPORTED = -8
CHAIN_MAX = 16
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1


class ChainLinear(ctypes.Structure):
    """``mt_chain_linear`` of include/minit_b200.h."""
    _fields_ = [("x", ctypes.c_void_p), ("qweight", ctypes.c_void_p), ("qzeros", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("n", ctypes.c_int), ("k", ctypes.c_int), ("nr_groups", ctypes.c_int), ("epilogue", ctypes.c_int),
                ("allreduce", ctypes.c_int)]

COUNTER_BYTES = 16384
STATIC_SCRATCH_BYTES = 8 << 20

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
#: every symbol include/minit_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "mt_version": (_i, []),
    "mt_strerror": (ctypes.c_char_p, [_i]),
    "mt_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "mt_dequant": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "mt_dequant_unpacked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "mt_unpack": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "mt_qgemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i]),
    "mt_qgemm_allreduce": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i, _vp, _i, _i, _sz]),
    "mt_qgemm_chain": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _sz, _i, _vp, _i, _i, _sz]),
    "mt_allreduce_buffer_bytes": (_sz, [_i, _i, _i]),
    "mt_qgemm_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i, _vp, _i, _i, _sz]),
    "mt_interleave_gate_up": (_i, [_vp] * 13 + [_i, _i, _i, _i]),
    "mt_qgemm_swiglu": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i]),
    "mt_swiglu": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "mt_rms_norm": (_i, [_vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _i]),
    "mt_rope_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _i]),
    "mt_qgemm_rope_append": (_i, [_vp] * 12 + [_i] * 8 + [_i, _vp, _i, _i, _vp, _sz, _i]),
    "mt_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, ctypes.c_float, _i]),
    "mt_attention_workspace_bytes": (_sz, [_i, _i, _i]),
    "mt_attention_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, ctypes.c_float, _vp, _sz, _i]),
    "mt_decode_plan": (_i, [_i, _i, _i, _i, _i, _sz, _i]),
    "mt_w8_pack": (_i, [_vp, _vp, _vp, _i, _i]),
    "mt_act_order_perm": (_i, [_vp, _vp, _vp, _vp, _i, _i]),
    "mt_repack_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "mt_gather_columns": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "mt_qgemm_ordered": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _i]),
    "mt_qgemm_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i]),
    "mt_w8_perchannel_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _i]),
    "mt_nccl_load": (_i, [ctypes.c_char_p]),
    "nccl_unique_id_size": (_sz, []),
    "nccl_create_unique_id": (_i, [_vp]),
    "nccl_init_rank": (_i, [_i, _i, _vp, _i, ctypes.POINTER(_vp)]),
    "nccl_destroy": (_i, [_vp]),
    "nccl_all_gather": (_i, [_vp, _vp, _vp, _vp, _sz, _i]),
    "nccl_all_reduce": (_i, [_vp, _vp, _vp, _vp, _sz, _i]),
    "nccl_broadcast": (_i, [_vp, _vp, _vp, _vp, _sz, _i, _i]),
}
for _name, (_res, _args) in SYMBOLS.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


class MinitError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status}: {lib.mt_strerror(status).decode()}")


def check(status: int, where: str) -> None:
    if status != 0:
        # argument errors map to ValueError like the reference's asserts, the rest to RuntimeError
        if status in (-1, -2, -3, -4, -5):
            raise ValueError(f"{where}: {lib.mt_strerror(status).decode()} (status {status})")
        raise MinitError(status, where)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return MT_F16
    if dtype == torch.bfloat16:
        return MT_BF16
    raise ValueError(f"unsupported dtype {dtype}: the quantized-linear kernels compute in float16 or bfloat16")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("minit_b200 kernels take CUDA tensors only (there is no CPU path)")
        if not t.is_contiguous():
            raise ValueError("minit_b200 kernels take contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors of one call must live on the same device")
    assert dev is not None
    return dev


# one zero-initialised workspace per (device, stream): the kernels keep the counter area zeroed
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        size = max(nbytes, 32 << 20)
        ws = torch.zeros(size, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def workspace_error_word(ws: torch.Tensor) -> int:
    """Error word a kernel sets when one of its bounded waits expires (4: a peer's all-reduce cells never arrived,
    5: an mbarrier wait of a tensor-core kernel).  Reading it synchronises with the device."""
    return int(ws[COUNTER_BYTES - 4:COUNTER_BYTES].view(torch.int32).item())


def raise_on_error_words(clear: bool = True) -> None:
    """Check the error word of every workspace of this process and raise ``MinitError`` (status
    ``ERR_PEER_TIMEOUT``) if a bounded device-side wait expired since the last check: the outputs of the
    calls in between are not valid (after an expired all-reduce wait the ranks no longer hold the same
    values).  It reads device memory, so call it where the host synchronises anyway -- after the read-back
    of a step's result, at the end of a benchmark step -- not per linear."""
    bad = []
    for key, ws in _workspaces.items():
        word = workspace_error_word(ws)
        if word:
            bad.append((key, word))
            if clear:
                ws[COUNTER_BYTES - 4:COUNTER_BYTES].zero_()
    if bad:
        err = MinitError(ERR_PEER_TIMEOUT, "bounded device-side wait")
        err.words = bad
        raise err
