from pfeife_b200.runtime.manager import PipeManager  # noqa: F401
