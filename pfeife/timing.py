from pfeife_b200.utils.timing import *  # noqa: F401,F403
from pfeife_b200.utils.timing import CPUEvent, CPUTimeRecorder, CUDATimeRecorder, TimeRecorder  # noqa: F401
