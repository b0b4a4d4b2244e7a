from pfeife_b200.topology import get_device, get_state, initialize_pfeife  # noqa: F401
from pfeife_b200.runtime.partial import PartialModule, PartialRunner, partial_compiler  # noqa: F401
from pfeife_b200.runtime.manager import PipeManager  # noqa: F401
