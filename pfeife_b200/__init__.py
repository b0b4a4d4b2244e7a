"""pfeife_b200: automatic pipeline-parallel training for one 8xB200 NVSwitch box.

Public surface (the reference's, pfeife/mp/__init__.py:1-8 and pfeife/option.py):
``initialize_pfeife``, ``get_state``, ``get_device``, ``PipeOption``, ``PartialRunner``,
``PartialModule``, ``partial_compiler``, ``PipeManager``; plus ``plan_mesh`` (the planner's
choice of the PP x DP mesh, which the reference leaves to ``--dp_mesh``).
"""
from .option import PipeOption  # noqa: F401
from .topology import get_device, get_state, initialize_pfeife  # noqa: F401


def __getattr__(name):
    # the runtime imports torch.distributed machinery; load it on first use
    if name in ("PartialRunner", "PartialModule", "partial_compiler", "worker_loop"):
        from .runtime import partial
        return getattr(partial, name)
    if name == "plan_mesh":
        from .parallel.mesh_plan import plan_mesh
        return plan_mesh
    if name == "PipeManager":
        from .runtime.manager import PipeManager
        return PipeManager
    raise AttributeError(name)
