from pfeife_b200.runtime.manager import LocalPipeManager as PipeManager  # noqa: F401
