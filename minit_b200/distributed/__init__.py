from .group import DistributedGroup, get_world, initialize_world, reset_world  # noqa: F401
from .communicator import DistributedCommunicator  # noqa: F401
