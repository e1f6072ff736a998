from . import symm_mem  # noqa: F401
from .health import Heartbeat, PeerLost  # noqa: F401
