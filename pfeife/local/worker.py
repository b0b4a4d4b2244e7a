from pfeife_b200.runtime.worker import StageWorker as ThreadWorker  # noqa: F401
