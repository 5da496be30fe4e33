from .library import connect_server, launch_server  # noqa: F401
from .tensor import NCCLTensor  # noqa: F401
from . import dispatch as _dispatch  # noqa: F401  registers the NCCL collectives
