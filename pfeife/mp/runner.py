"""``pfeife.mp.runner`` of the reference (pfeife/mp/runner.py:30-300) holds the compiled-module
wrapper of its manager front-end (``PipeGraphRunner``) and the thread pool that runs one
micro-batch per thread (``RunnerThreadPool``).  Here both roles belong to the partial runtime:
the captured module is a ``PartialModule`` and the micro-batch threads are owned by
``PartialRunner``."""
from pfeife_b200.runtime.partial import PartialModule, PartialRunner  # noqa: F401

PipeGraphRunner = PartialModule
RunnerThreadPool = PartialRunner
