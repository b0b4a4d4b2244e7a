"""Choosing the PP x DP mesh before the job's process groups exist.

The mesh fixes which ranks form a pipeline and which are replicas, so it has to be known when
``initialize_pfeife`` builds the process groups.  ``plan_mesh`` runs on ONE process with one
device: it captures the model's FX graph, profiles it with one micro-batch (the same
segment-by-segment pass the runner uses), and evaluates every factorisation of the world size
with the planner's cost model (pipeline makespan + exposed data-parallel time) under the
device's memory.  The reference leaves this choice to the user's ``--dp_mesh``
(pfeife/mp/partial/runner.py:32-106 takes the mesh as given); here it is the planner's call.
"""
from __future__ import annotations

import copy
from typing import Any, Optional, Sequence

import torch

from ..graph.capture import classify_inputs
from ..graph.profiler import gen_comp_graph_cpu, gen_local_comp_graph
from ..utils import get_logger
from .device_bench import DeviceBench
from .planner import MeshChoice, choose_mesh

# NVLink 5 through NVSwitch, every pair alike: 0.02 ms to start a transfer, 770 GB/s after that
NVSWITCH_LINK = (0.02, 1.0 / 770e3, 0.0)


class _Probe(torch.nn.Module):
    """Compile backend product that remembers the flat call arguments of the captured graph."""

    def __init__(self, gm, example_inputs):
        super().__init__()
        self.gm = gm
        self.example_inputs = example_inputs
        self.args: Optional[Sequence[Any]] = None

    def forward(self, *args):
        if self.args is None:
            self.args = args
        return self.gm(*args)


def plan_mesh(model: torch.nn.Module, micro_batch: Sequence[Any], option, world_size: int,
              device: Optional[torch.device] = None,
              link: Sequence[float] = NVSWITCH_LINK) -> MeshChoice:
    """Profile `model` on `device` with the tensors of one micro-batch and return the best
    ``MeshChoice`` (``.pp``, ``.dp``, ``.dp_mesh`` string for ``initialize_pfeife``) for
    `world_size` devices.  `option` supplies batch_size / batch_cnt / mixed precision /
    partitioner / scheduler exactly as it will for training."""
    log = get_logger()
    device = torch.device(device) if device is not None else next(model.parameters()).device
    probes = []

    def backend(gm, example_inputs):
        p = _Probe(gm, example_inputs)
        probes.append(p)
        return p

    import torch._dynamo as dynamo
    dynamo.reset()
    compiled = torch.compile(model, backend=backend)
    with torch.no_grad():
        compiled(*micro_batch)
    dynamo.reset()
    probes = [p for p in probes if p.args is not None]
    if not probes:
        raise RuntimeError("the model produced no graph to plan")
    # the first graph with parameters is the one the runner would pipeline
    probe = next((p for p in probes if any(isinstance(a, torch.nn.Parameter) for a in p.args)),
                 probes[0])
    captured = classify_inputs(probe.gm, probe.example_inputs)
    opt = copy.copy(option)
    opt.graph_bench = None
    if device.type == "cuda":
        cg, _ = gen_local_comp_graph(captured, probe.args, device, opt)
        mem = float(torch.cuda.get_device_properties(device).total_memory)
    else:
        cg, _ = gen_comp_graph_cpu(captured, probe.args, opt)
        mem = float(64 << 30)
    bench = DeviceBench()
    bench.set_uniform(world_size, tuple(link))
    choice = choose_mesh(cg, world_size, opt, bench, mem)
    log.info("plan_mesh: PP=%d x DP=%d for %d devices", choice.pp, choice.dp, world_size)
    return choice
