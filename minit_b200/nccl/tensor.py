"""The 0-d "version token" that carries the NCCL communicator through dispatch
(reference: minit/nccl/tensor.py:5-27)."""
from .library import connect_server


class NCCLTensor:
    def __init__(self, comm: int) -> None:
        self.comm = comm

    @property
    def shape(self):
        return ()

    @property
    def dtype(self):
        return "int64"

    @property
    def device(self):
        return "nccl"

    @staticmethod
    def connect(unique_id: bytes, rank: int, size: int, device=None) -> "NCCLTensor":
        return NCCLTensor(connect_server(size, rank, unique_id, device))
