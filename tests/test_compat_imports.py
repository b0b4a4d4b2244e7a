"""A script written against the reference's import paths (``pfeife.*``) finds the same names."""
import importlib

import pytest

SURFACE = {
    "pfeife.option": ["PipeOption"],
    "pfeife.mp": ["initialize_pfeife", "get_state", "get_device", "PartialRunner", "PartialModule",
                  "partial_compiler", "PipeManager"],
    "pfeife.mp.partial": ["PartialRunner", "PartialModule", "partial_compiler"],
    "pfeife.mp.partial.module": ["PartialRunner", "PartialModule", "partial_compiler"],
    "pfeife.mp.manager": ["PipeManager"],
    "pfeife.mp.runner": ["PipeGraphRunner", "RunnerThreadPool"],
    "pfeife.mp.worker": ["ProcessWorker", "LoopFlag"],
    "pfeife.mp.net_states": ["PfeifeState", "initialize_pfeife", "get_state", "get_device",
                             "get_pp_rank", "get_global_rank", "get_pp_group_ranks",
                             "get_dp_group_ranks", "check_main_rank", "target_main_rank"],
    "pfeife.local.manager": ["PipeManager"],
    "pfeife.local.runner": ["LocalRunner", "LocalReducer"],
    "pfeife.local.worker": ["ThreadWorker"],
    "pfeife.local.graph_bench": ["gen_comp_graph", "gen_comp_graph_cpu", "gen_amp_context"],
    "pfeife.schedule.planner": ["PipeGraphGenerator", "BeamSearchGenerator", "BeamSingleGenerator",
                                "DependencyGraph", "get_pipe_class"],
    "pfeife.schedule.scheduler": ["PipeSchedParams", "PipeSchedSet", "Scheduler", "BeamScheduler",
                                  "BFSScheduler", "DFSScheduler", "PipelessScheduler",
                                  "NoSkewScheduler", "SingleCommScheduler", "Step", "StepWork"],
    "pfeife.schedule.solver": [],
    "pfeife.graph.computation_graph": ["CompGraph", "CompNode", "CompEdge"],
    "pfeife.graph.partition_graph": ["PartitionGraph"],
    "pfeife.graph.pipe_graph": ["PipeGraph", "PipeNode", "PipeEdge"],
    "pfeife.device_bench": ["DeviceBench", "NCCLDeviceBench"],
    "pfeife.loss": ["LossWrapper", "CrossEntropyLoss", "HFCrossEntropyLoss", "MaskedLMOutputLoss",
                    "SumLoss", "RescaleLoss", "NormalizeLoss"],
    "pfeife.batch": ["split_args_kwargs"],
    "pfeife.timing": ["CUDATimeRecorder", "CPUTimeRecorder", "TimeRecorder"],
    "pfeife.utils": ["get_logger", "set_logger_level", "set_seed", "to_device", "fmem", "Recorder",
                     "tree_trav", "tree_filter"],
    "pfeife.compile": ["compile_module"],
}


@pytest.mark.parametrize("module", sorted(SURFACE))
def test_reference_import_path(module):
    mod = importlib.import_module(module)
    missing = [n for n in SURFACE[module] if not hasattr(mod, n)]
    assert not missing, f"{module} lacks {missing}"
    if module.startswith("pfeife.mp") and hasattr(mod, "PartialRunner"):
        from pfeife_b200.runtime.partial import PartialRunner
        assert mod.PartialRunner is PartialRunner
