from pfeife_b200.runtime.worker import LoopFlag, StageWorker  # noqa: F401
from pfeife_b200.runtime.partial import worker_loop  # noqa: F401

ProcessWorker = StageWorker
