"""Process-level plumbing: control plane, communicator, symmetric memory, local launcher."""
from .bootstrap import Bootstrap  # noqa: F401
from .symmetric import Communicator, DeviceStatus, DeviceWaitError, SymmetricBuffer  # noqa: F401
