"""NCCL bootstrap (reference: minit/nccl/library.py:41-101): ``launch_server()`` makes the
unique id on one rank, ``connect_server(nr_ranks, rank, id)`` joins the communicator.  The
id travels between ranks by whatever control plane the launcher has (the reference uses a
file or its TCP controller; under torchrun use torch.distributed's store, see
``exchange_unique_id``)."""
from __future__ import annotations

import ctypes
import os

from .. import _lib

_loaded = False


def _ensure_loaded() -> None:
    """Open the same libnccl torch ships with, so one process never holds two NCCL copies."""
    global _loaded
    if _loaded:
        return
    path = os.environ.get("MINIT_B200_NCCL")
    if path is None:
        try:
            import nvidia.nccl
            cand = os.path.join(list(nvidia.nccl.__path__)[0], "lib", "libnccl.so.2")
            path = cand if os.path.exists(cand) else None
        except ImportError:
            path = None
    _lib.check(_lib.lib.mt_nccl_load(path.encode() if path else None), "mt_nccl_load")
    _loaded = True


def launch_server() -> bytes:
    _ensure_loaded()
    size = _lib.lib.nccl_unique_id_size()
    buf = ctypes.create_string_buffer(size)
    _lib.check(_lib.lib.nccl_create_unique_id(ctypes.cast(buf, ctypes.c_void_p)), "nccl_create_unique_id")
    return bytes(buf.raw)


def connect_server(nr_ranks: int, rank: int, id: bytes, device: int | None = None) -> int:
    """Join the communicator; the reference binds rank r to device r (minit/nccl/library.py:53-56),
    which stays the default."""
    _ensure_loaded()
    assert len(id) == _lib.lib.nccl_unique_id_size()
    comm = ctypes.c_void_p()
    buf = ctypes.create_string_buffer(id, len(id))
    _lib.check(_lib.lib.nccl_init_rank(nr_ranks, rank, ctypes.cast(buf, ctypes.c_void_p),
                                       rank if device is None else device, ctypes.byref(comm)), "nccl_init_rank")
    return comm.value


def exchange_unique_id(rank: int) -> bytes:
    """Share rank 0's unique id through the torch.distributed store of an initialised process group."""
    import torch.distributed as dist
    box = [launch_server() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]
