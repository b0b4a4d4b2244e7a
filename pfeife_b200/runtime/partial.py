"""Public training front-end: ``partial_compiler`` (a ``torch.compile`` backend),
``PartialModule`` and ``PartialRunner(option, optimizer).set_exec_fn / step``.

User contract (pfeife/mp/partial/module.py:37-438, README "How to train custom models"):

    initialize_pfeife()
    option = PipeOption.from_args(args)
    runner = PartialRunner(option, optimizer)
    model = torch.compile(model, backend=partial_compiler)
    runner.set_exec_fn(iter_fn)          # iter_fn(micro_batch...) calls model, loss.backward()
    losses = runner.step(batch)          # one optimizer step over batch_cnt micro-batches

``exec_fn`` runs in ``batch_cnt`` threads, one per micro-batch.  The compiled model call inside
it lands in ``PartialModule.forward``, which hands the micro-batch's inputs to the pipeline,
blocks until the last stage produced that micro-batch's outputs and returns them as detached
leaves whose gradient hooks feed the pipeline's backward.  The first ``step`` probes (captures
and profiles the graph with micro-batch 0), plans, partitions and distributes.

Ranks that are not the main rank of their pipeline run ``worker_loop()`` instead of the user
script (``mp_launch.py`` does this for them).
"""
from __future__ import annotations

import atexit
import contextlib
import copy
import os
import queue
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..graph.capture import CapturedGraph, classify_inputs
from ..graph.comp_graph import CompGraph
from ..graph.partition import PartitionGraph, partition_module
from ..graph.profiler import gen_comp_graph_cpu, gen_local_comp_graph, run_unprofiled
from ..option import PipeOption
from ..parallel.device_bench import DeviceBench, NCCLDeviceBench
from ..parallel.planner import Plan, get_pipe_class
from ..parallel.schedule import get_scheduler_class
from ..topology import PfeifeState, get_state
from ..utils import get_logger
from ..utils.batch import split_args_kwargs
from .params import StateEntry, snapshot_hyper
from .transport import DistTransport
from .worker import LoopFlag, StageWorker

STEP_TOKEN = object()
_tls = threading.local()
_current_runner: Optional["PartialRunner"] = None


# ------------------------------------------------------------------------------ control plane
# entry of the optimizer-state dictionary that carries the job's loss scale (not a parameter name)
SCALER_KEY = "__loss_scaler__"


class ControlPlane:
    """Small host-side messages between the ranks of one pipeline (gloo)."""

    def __init__(self, state: PfeifeState):
        self.state = state
        self.group = state.ctrl_pp
        self.src = state.pp_main_rank

    def bcast(self, obj: Any = None) -> Any:
        if self.state.pp_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    def gather(self, obj: Any) -> Optional[List[Any]]:
        if self.state.pp_size == 1:
            return [obj]
        out = [None] * self.state.pp_size if self.state.rank == self.src else None
        dist.gather_object(obj, out, dst=self.src, group=self.group)
        return out

    def scatter(self, objs: Optional[List[Any]]) -> Any:
        """Main rank passes one object per pp rank; every rank returns its own."""
        if self.state.pp_size == 1:
            return objs[0]
        out = [None]
        dist.scatter_object_list(out, objs if self.state.rank == self.src else None,
                                 src=self.src, group=self.group)
        return out[0]

    def barrier(self) -> None:
        if self.state.pp_size > 1:
            dist.barrier(group=self.group)

    def share_with_replicas(self, obj: Any = None) -> Any:
        """Main ranks only: the object of the first replica's main rank, on every replica's main
        rank.  The main ranks of all pipelines hold the same pipeline rank, so together they are
        one data-parallel group."""
        if self.state.dp_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self.state.dp_group_ranks[0], group=self.state.ctrl_dp)
        return box[0]


class _DistReducer:
    def __init__(self, group):
        self.group = group

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)


def _make_worker(state: PfeifeState, option: PipeOption, runner=None) -> StageWorker:
    transport = None
    if state.pp_size > 1:
        transport = DistTransport(state.rank, state.layout.all_pp_groups(), state.device)
    w = StageWorker(state.pp_rank, state.pp_size, state.device, option, transport, runner,
                    global_ranks=state.pp_group_ranks)

    def sync_found_inf():
        if state.world_size > 1:
            dist.all_reduce(w.params.found_inf, op=dist.ReduceOp.MAX)
    w.sync_found_inf = sync_found_inf
    if state.dp_size > 1:
        from ..parallel.dp import make_dp
        w.dp = make_dp(state, option)
    return w


def _install_plan(worker: StageWorker, state: PfeifeState, payload: Dict[str, Any]) -> None:
    worker.batch_cnt = payload["batch_cnt"]
    worker.set_partition_graph(payload["part"], payload["entries"], payload["optimizer_type"],
                               payload["hyper"])
    worker.set_scheduler_steps(payload["steps"], payload["eval_steps"])
    # groups for parameters shared across pipeline ranks: every rank of the job creates every
    # group, in the same order
    sets = sorted({tuple(r) for r in payload["part"].shared_states.values()})
    made: Dict[Tuple[int, ...], Any] = {}
    for pp_ranks in sets:
        for pipeline in state.layout.all_pp_groups():
            ranks = [pipeline[r] for r in pp_ranks]
            g = dist.new_group(ranks)
            if state.rank in ranks:
                made[pp_ranks] = _DistReducer(g)
    worker.shared_groups = {k: v for k, v in made.items() if worker.pp_rank in k}


def worker_loop(option: Optional[PipeOption] = None) -> None:
    """Body of a non-main pipeline rank (pfeife/mp/worker.py:168-240 ``wait_for_init`` +
    ``run_loop``): receive the options and the plan, then execute step programs until told to
    stop."""
    state = get_state()
    ctrl = ControlPlane(state)
    option = ctrl.bcast(None)
    option.set_logger()
    worker = _make_worker(state, option)
    _run_device_bench(state, option)
    payload = ctrl.scatter(None)
    if payload.get("abort"):        # the main rank failed before it had a plan
        return
    _install_plan(worker, state, payload)
    ctrl.barrier()
    while True:
        msg = ctrl.bcast(None)
        flag = msg["flag"]
        if flag == LoopFlag.STOP_LOOP:
            break
        if flag in (LoopFlag.CONTINUE_LOOP, LoopFlag.EVAL_LOOP):
            worker.reset_cache()
            worker.params.set_hyper(msg.get("hyper"))
            worker.run(training=(flag == LoopFlag.CONTINUE_LOOP))
        elif flag == LoopFlag.GATHER_PARAMS:
            named = {k: v.cpu() for k, v in worker.params.named_tensors().items()}
            opt = {k: {kk: vv.cpu() for kk, vv in st.items()}
                   for k, st in worker.params.optimizer_state().items()} if msg.get("opt") else {}
            if msg.get("opt") and worker.scaler.enabled:
                opt[SCALER_KEY] = worker.scaler.state_dict()
            ctrl.gather((named, opt))
        elif flag == LoopFlag.LOAD_PARAMS:
            worker.params.load_named(msg["named"])
            if msg.get("opt"):
                worker.params.load_optimizer_state(msg["opt"])
                worker.scaler.load_state_dict(msg["opt"].get(SCALER_KEY))
        elif flag == LoopFlag.LOG_MEMORY_USAGE:
            worker.log_memory_usage()
        elif flag == LoopFlag.REPORT_TIMES:
            rep = worker.time_report(msg.get("reset", True))
            rep["memory"] = worker.memory_usage()
            ctrl.gather(rep)


def _run_device_bench(state: PfeifeState, option: PipeOption) -> DeviceBench:
    """Link model shared by the ranks of a pipeline; measured once or loaded from
    ``option.device_bench`` (pfeife/mp/worker.py:242-263)."""
    if state.pp_size == 1:
        return DeviceBench()
    bench = NCCLDeviceBench(state.rank, state.pp_group_ranks, state.device, state.pp_group, option)
    if state.cpu and not (option.device_bench and os.path.exists(option.device_bench)):
        bench.set_uniform(state.pp_size, (0.05, 1.0, 0.0))   # CPU runs: a fixed toy link
    else:
        bench.run_bench(option.device_bench, uniform=True)
    return bench


# ------------------------------------------------------------------------------ PartialModule
class PartialModule(torch.nn.Module):
    """One captured FX graph.  Pipelined when it is the first eligible graph of the model
    (enough compute nodes for ``pp_size`` stages); any other graph runs locally as captured
    (pfeife/mp/partial/module.py:205-216, 392-396)."""

    def __init__(self, gm: torch.fx.GraphModule, example_inputs: Sequence[Any]):
        super().__init__()
        self.gm = gm
        self.runner: Optional[PartialRunner] = _current_runner
        self.captured: Optional[CapturedGraph] = None
        self.should_pp = False
        self.probed = False
        self.compiled = False
        self.comp_graph: Optional[CompGraph] = None
        self.part: Optional[PartitionGraph] = None
        self.plan: Optional[Plan] = None
        if self.runner is not None:
            self.captured = classify_inputs(gm, example_inputs)
            pp = self.runner.state.pp_size
            n_nodes = self.captured.compute_node_count()
            already = any(m.should_pp for m in self.runner.modules)
            # the reference's rule (pfeife/mp/partial/module.py:205-216): at least 2*pp graph
            # nodes, of which at least pp compute; parameters are placeholders here and do not
            # count as graph nodes
            n_graph = n_nodes + len(self.captured.user_inputs) + 1
            self.should_pp = (not already) and n_graph >= 2 * pp and n_nodes >= pp and \
                len(self.captured.params) > 0
            self.pipe_idx = len(self.runner.modules)
            self.runner.modules.append(self)
            # buffers that a forward pass updates (BatchNorm statistics and the like): the
            # profiling passes below run the graph several times on the real tensors, and
            # training must start from the values the user handed over, not from those
            self._buffers_at_capture = {gi.index: gi.tensor.detach().clone()
                                        for gi in self.captured.buffers} if self.should_pp else {}

    # -- first call: profile on the main rank, return a real output so exec_fn can continue
    def _probe_forward(self, args: Sequence[Any]) -> Any:
        """One profile per job.  With data parallelism every replica's main rank captures the
        same graph, but only the first replica measures it; its per-segment statistics go to the
        other replicas, which run the graph once for the output their ``exec_fn`` continues
        with.  Replicas that profiled on their own would see different timings, could choose
        different split points and would then disagree on buffer layouts and group creation
        (the reference shares one profile file, pfeife/mp/partial/module.py:263-272)."""
        r = self.runner
        opt, state = r.option, r.state
        if state.dp_size == 1 or state.dp_rank == 0:
            if state.cpu:
                cg, out = gen_comp_graph_cpu(self.captured, args, opt)
            else:
                cg, out = gen_local_comp_graph(self.captured, args, state.device, opt)
            r.ctrl.share_with_replicas(cg.graph_data())
        else:
            cg, out = run_unprofiled(self.captured, args, state.device, opt)
            cg.apply_graph_data(r.ctrl.share_with_replicas(None))
        self.comp_graph = cg
        self.probed = True
        return out

    def _compile(self, optimizer) -> None:
        """Plan, partition and distribute (pfeife/mp/partial/module.py:290-371)."""
        r = self.runner
        opt, state = r.option, r.state
        with torch.no_grad():
            for gi in self.captured.buffers:
                saved = self._buffers_at_capture.get(gi.index)
                if saved is not None:
                    gi.tensor.copy_(saved)
        self._buffers_at_capture = {}
        pp = state.pp_size
        opt_pp = copy.copy(opt)
        opt_pp.device_cnt = pp
        if pp == 1:
            opt_pp.loop_cnt = 1
        max_mem = None
        if state.device.type == "cuda":
            total = torch.cuda.get_device_properties(state.device).total_memory
            max_mem = [float(total)] * pp
        gen = get_pipe_class(opt.partitioner)(self.comp_graph, r.device_bench, opt_pp)
        # one search per job: the first replica's split points and schedule parameters are
        # installed by every replica (their link measurements differ, their plans must not)
        if state.dp_size == 1 or state.dp_rank == 0:
            plan = gen.gen_graph(opt.batch_cnt, max_mem, opt.split_points)
            r.ctrl.share_with_replicas((list(plan.split_points), plan.sched.key()))
        else:
            points, sched_key = r.ctrl.share_with_replicas(None)
            plan = gen.plan_from(points, sched_key, max_mem)
        self.plan = plan
        if getattr(opt, "schedule_picture", None) and state.is_main_process:
            from ..parallel.gantt import save_schedule_svg
            save_schedule_svg(plan.pipe_graph, plan.sched, opt.schedule_picture, plan.sim)
        part = partition_module(self.comp_graph, plan.split_points, pp)
        self.part = part
        sched_cls = get_scheduler_class(opt.scheduler)
        sched = sched_cls(plan.sched, plan.dep_graph)
        steps = sched.steps
        eval_steps = [sched.get_eval_steps(i) for i in range(pp)]

        # parameter entries per rank, with the user's optimizer group of every parameter
        group_of: Dict[int, int] = {}
        if optimizer is not None:
            for gi, g in enumerate(optimizer.param_groups):
                for p in g["params"]:
                    group_of[id(p)] = gi
        hyper = snapshot_hyper(optimizer) if optimizer is not None else \
            [dict(opt.optimizer_kwargs)]
        opt_type = type(optimizer).__name__ if optimizer is not None else opt.optimizer_type
        shadow_only = self.captured.shadow_only_inputs()
        payloads = []
        for rank in range(pp):
            entries = []
            for ph in part.rank_states(rank):
                gi = self.captured.inputs[ph]
                t = gi.tensor
                entries.append(StateEntry(ph, gi.qualname, gi.kind,
                                          t.detach() if rank == state.pp_rank else t.detach().cpu(),
                                          bool(gi.kind == "param" and t.requires_grad),
                                          group_of.get(id(t), 0), lp_only=(ph in shadow_only)))
            payloads.append({"part": part.for_rank(rank), "entries": entries,
                             "optimizer_type": opt_type, "hyper": hyper, "steps": steps,
                             "eval_steps": eval_steps, "batch_cnt": opt.batch_cnt})
        mine = r.ctrl.scatter(payloads)
        r.install_plan(mine)
        r.ctrl.barrier()
        self.compiled = True
        # the user's module keeps its Parameter objects; they are refreshed by gather_params()
        for gi in self.captured.params:
            gi.tensor.grad = None

    def forward(self, *args):
        r = self.runner
        if r is None or not self.should_pp:
            return self.gm(*args)
        if not self.probed:
            return self._probe_forward(args)
        if not self.compiled:      # probe call of a later graph while the first is compiling
            return self.gm(*args)
        return self._wait_for_execution(args)

    def _wait_for_execution(self, args: Sequence[Any]) -> Any:
        r = self.runner
        mb = getattr(_tls, "mb", None)
        if mb is None:
            raise RuntimeError("the compiled model must be called from exec_fn inside "
                               "PartialRunner.step()")
        values = {gi.index: args[gi.index] for gi in self.captured.user_inputs}
        r.worker.submit_inputs(mb, values)
        r._return_queues[mb].put(STEP_TOKEN)           # "my inputs are in"
        outs = r._module_queues[mb].get()              # blocks until the last stage ran
        if isinstance(outs, BaseException):
            raise outs
        return self.part.assemble_output(outs, args)


def partial_compiler(gm: torch.fx.GraphModule, example_inputs: Sequence[Any]) -> PartialModule:
    """``torch.compile(model, backend=partial_compiler)``."""
    return PartialModule(gm, example_inputs)


# ------------------------------------------------------------------------------ PartialRunner
class PartialRunner:
    def __init__(self, option: PipeOption, optimizer=None):
        global _current_runner
        self.option = option
        self.optimizer = optimizer
        self.log = get_logger()
        self.modules: List[PartialModule] = []
        self.exec_fn: Optional[Callable] = None
        self.batch_cnt = option.batch_cnt
        _current_runner = self
        self._setup_runtime()
        self._start_threads()

    def _setup_runtime(self) -> None:
        """Process-per-GPU runtime: topology from ``initialize_pfeife``, control plane over
        gloo, one StageWorker for this rank."""
        option = self.option
        self.state = get_state()
        if not self.state.is_main_rank:
            raise RuntimeError("PartialRunner belongs to the main rank of a pipeline; other "
                               "ranks call worker_loop() (mp_launch.py does)")
        self.ctrl = ControlPlane(self.state)
        self.ctrl.bcast(option)
        self.worker = _make_worker(self.state, option, runner=self)
        self.device_bench = _run_device_bench(self.state, option)

    def install_plan(self, payload: Dict[str, Any]) -> None:
        _install_plan(self.worker, self.state, payload)

    def _start_threads(self) -> None:
        self._train_queues = [queue.Queue() for _ in range(self.batch_cnt)]
        self._return_queues = [queue.Queue() for _ in range(self.batch_cnt)]
        self._module_queues = [queue.Queue() for _ in range(self.batch_cnt)]
        self._threads = []
        for bid in range(self.batch_cnt):
            t = threading.Thread(target=self._exec_loop, args=(bid,), daemon=True)
            t.start()
            self._threads.append(t)
        self._closed = False
        self._compiled = False
        self._pending_load = None
        atexit.register(self.close)

    # ---- user API
    def set_exec_fn(self, fn: Callable) -> None:
        self.exec_fn = fn

    @property
    def scaler(self):
        """The job-wide loss scaler: ``runner.scaler.scale(loss).backward()`` under fp16."""
        return self.worker.scaler

    def step(self, *args, **kwargs) -> List[Any]:
        if self.exec_fn is None:
            raise RuntimeError("call set_exec_fn() before step()")
        a_split, k_split = split_args_kwargs(args, kwargs, self.batch_cnt)
        if not self._compiled:
            try:
                self._probe_forward(a_split[0], k_split[0])
                pipelined = [m for m in self.modules if m.should_pp and m.probed]
                if not pipelined:
                    raise RuntimeError("no captured graph is eligible for pipelining: the model "
                                       "call must happen inside exec_fn and the graph needs at "
                                       f"least {self.state.pp_size} compute nodes")
                for m in pipelined:
                    m._compile(self.optimizer)
            except BaseException:
                self._release_workers()
                raise
            self._compiled = True
            if self._pending_load is not None:     # a checkpoint handed over before the first step
                named, opt = self._pending_load
                self._pending_load = None
                self.load_params(named, opt)
        return self._run(a_split, k_split, training=True)

    def _release_workers(self) -> None:
        """The first step failed before the plan went out: the other ranks of the pipeline are
        still waiting for it.  They get an empty plan, which ends their loop, and this runner is
        closed, so that the error surfaces instead of a stalled job."""
        if self._closed:
            return
        self._closed = True
        if not any(m.compiled for m in self.modules):
            try:
                self.ctrl.scatter([{"abort": True}] * self.state.pp_size)
            except Exception:
                pass
        for q in self._train_queues:
            q.put(None)

    def eval_step(self, *args, **kwargs) -> List[Any]:
        """Forward-only pass through the pipeline; exec_fn must not call backward."""
        a_split, k_split = split_args_kwargs(args, kwargs, self.batch_cnt)
        if not self._compiled:
            raise RuntimeError("run one training step before eval_step()")
        return self._run(a_split, k_split, training=False)

    def _run(self, a_split, k_split, training: bool) -> List[Any]:
        self.reset(training)
        self._training = training
        for bid in range(self.batch_cnt):
            self._train_queues[bid].put((a_split[bid], k_split[bid]))
        for bid in range(self.batch_cnt):      # every thread reached the model call
            tok = self._return_queues[bid].get(timeout=self.option.ctrl_timeout)
            if tok is not STEP_TOKEN:
                self._abort(tok)
        try:
            self.worker.run(training)
        except BaseException as e:
            for q in self._module_queues:
                q.put(e)
            raise
        results = []
        for bid in range(self.batch_cnt):
            res = self._return_queues[bid].get(timeout=self.option.ctrl_timeout)
            if isinstance(res, BaseException):
                raise res
            results.append(res)
        return results

    def _abort(self, tok):
        if isinstance(tok, BaseException):
            raise tok
        raise RuntimeError("exec_fn returned without calling the compiled model")

    def reset(self, training: bool = True) -> None:
        self.worker.reset_cache()
        msg = {"flag": LoopFlag.CONTINUE_LOOP if training else LoopFlag.EVAL_LOOP}
        if self.optimizer is not None:
            msg["hyper"] = snapshot_hyper(self.optimizer)
            self.worker.params.set_hyper(msg["hyper"])
        self.ctrl.bcast(msg)

    # ---- outputs and loss gradients (called from the worker / the batch threads)
    def return_output(self, mb: int, stage: int, sink: List[Tuple[int, torch.Tensor]]) -> None:
        outs: Dict[Tuple[int, int], Any] = {}
        training = getattr(self, "_training", True)
        for j, t in sink:
            if torch.is_tensor(t):
                leaf = t.detach()
                if training and t.requires_grad and leaf.dtype.is_floating_point:
                    leaf.requires_grad_(True)
                    leaf.register_hook(self._make_hook(mb, j))
                outs[(stage, j)] = leaf
            else:
                outs[(stage, j)] = t
        self._module_queues[mb].put(outs)

    def _make_hook(self, mb: int, j: int):
        def hook(grad):
            self.worker.recv_loss_grad(mb, j, grad)
            return grad
        return hook

    def finalize_output(self, mb: int) -> None:
        self.worker.loss_backward_done(mb)

    # ---- threads
    def _exec_loop(self, bid: int) -> None:
        _tls.mb = bid
        if self.state.device.type == "cuda":
            torch.cuda.set_device(self.state.device)   # new threads start on device 0
        while True:
            item = self._train_queues[bid].get()
            if item is None:
                return
            a, k = item
            try:
                with self._amp():
                    res = self.exec_fn(*a, **k)
            except BaseException as e:   # surfaced by step()
                self._return_queues[bid].put(e)
                self.finalize_output(bid)
                continue
            self.finalize_output(bid)
            self._return_queues[bid].put(res)

    def _probe_forward(self, a, k) -> Any:
        _tls.mb = None
        with self._amp():
            res = self.exec_fn(*a, **k)
        return res

    def _amp(self):
        """The user's step function runs under the same autocast state as the stages: the graph
        is traced inside it, and dtypes that the trace bakes in (``t.to(x.dtype)``) must be the
        ones the stages will see.  (The stages enter autocast themselves,
        pfeife/mp/worker.py:677; tracing outside it gives fp32 where they produce 16 bits.)"""
        from ..graph.profiler import gen_amp_context
        from ..ops import functional as Fn
        stack = contextlib.ExitStack()
        stack.enter_context(gen_amp_context(self.state.device, self.option.mixed_precision))
        # meta functions of a trace run with autocast off: tell them the stages' precision
        stack.enter_context(Fn.stage_precision(self.option.mixed_precision))
        return stack

    # ---- checkpoint
    def gather_params(self, with_optimizer: bool = False):
        """Copies every rank's current parameters back into the user's module (so that
        ``model.state_dict()`` is a plain checkpoint of the original module,
        pfeife/mp/partial/module.py:115-117) and, optionally, returns the optimizer state keyed
        by the original parameter names."""
        self.ctrl.bcast({"flag": LoopFlag.GATHER_PARAMS, "opt": with_optimizer})
        named = {k: v for k, v in self.worker.params.named_tensors().items()}
        opt = self.worker.params.optimizer_state() if with_optimizer else {}
        gathered = self.ctrl.gather((named, opt)) if self.state.pp_size > 1 else [(named, opt)]
        all_named: Dict[str, torch.Tensor] = {}
        all_opt: Dict[str, Dict[str, torch.Tensor]] = {}
        mine = self.worker.scaler.state_dict() if self.worker.scaler.enabled else None
        for item in gathered:
            if item is None:
                continue
            all_named.update(item[0])
            theirs = item[1].pop(SCALER_KEY, None) if isinstance(item[1], dict) else None
            if theirs is not None and mine is not None and \
                    float(theirs["scale"]) != float(mine["scale"]):
                raise RuntimeError(
                    f"the loss scale differs between pipeline ranks ({float(theirs['scale'])} vs "
                    f"{float(mine['scale'])}): a rank skipped a step that another applied")
            all_opt.update(item[1])
        all_named.update(named)
        all_opt.update(opt)
        if with_optimizer and mine is not None:
            all_opt[SCALER_KEY] = mine      # one scale for the whole job
        with torch.no_grad():
            for m in self.modules:
                if not m.should_pp:
                    continue
                for gi in m.captured.inputs:
                    if gi.is_state and gi.qualname in all_named:
                        gi.tensor.copy_(all_named[gi.qualname].to(gi.tensor.device))
        return all_opt if with_optimizer else None

    def load_params(self, named: Dict[str, torch.Tensor],
                    opt: Optional[Dict[str, Dict[str, torch.Tensor]]] = None) -> None:
        """Resume: pushes a ``state_dict`` of the original module (and optimizer state) to the
        ranks that own each parameter.  Before the first step no rank owns anything yet: the
        checkpoint is kept and applied as soon as the stages exist, before that step computes."""
        named = {k: v.detach().cpu() for k, v in named.items()}
        if not self._compiled:
            self._pending_load = (named, opt)
            return
        self.ctrl.bcast({"flag": LoopFlag.LOAD_PARAMS, "named": named, "opt": opt})
        self.worker.params.load_named(named)
        if opt:
            self.worker.params.load_optimizer_state(opt)
            self.worker.scaler.load_state_dict(opt.get(SCALER_KEY))

    def log_memory_usage(self) -> None:
        self.ctrl.bcast({"flag": LoopFlag.LOG_MEMORY_USAGE})
        self.worker.log_memory_usage()

    def time_report(self, reset: bool = True) -> List[Dict[str, Any]]:
        """Per pipeline rank of this pipeline: device time spent in stage forwards, backwards
        and optimizer steps since the last report, the number of steps covered and the memory
        figures (``StageWorker.time_report``).  ``bubble_report`` turns it into idle shares."""
        self.ctrl.bcast({"flag": LoopFlag.REPORT_TIMES, "reset": reset})
        mine = self.worker.time_report(reset)
        mine["memory"] = self.worker.memory_usage()
        reps = self.ctrl.gather(mine) if self.state.pp_size > 1 else [mine]
        return [r for r in reps if r is not None]

    def bubble_report(self, step_ms: float, reset: bool = True) -> Dict[str, Any]:
        """Measured pipeline bubble of the steps since the last report, given their mean
        device time: per rank ``1 - (forward + backward time) / (step time - optimizer time)``,
        with the maximum and mean over the ranks of this pipeline (the reference records the
        same per-stage events and never reads them back, pfeife/mp/worker.py:1484-1499)."""
        per_rank = []
        for r in sorted(self.time_report(reset), key=lambda r: r["pp_rank"]):
            n = max(1, r["steps"])
            busy = (r["fwd_ms"] + r["bwd_ms"]) / n
            window = max(step_ms - r["opt_ms"] / n, 1e-9)
            per_rank.append({"pp_rank": r["pp_rank"], "busy_ms": busy, "opt_ms": r["opt_ms"] / n,
                             "bubble_pct": 100.0 * max(0.0, 1.0 - busy / window),
                             "max_mem_bytes": r["memory"]["max"]})
        b = [r["bubble_pct"] for r in per_rank]
        return {"per_rank": per_rank, "max_pct": max(b), "mean_pct": sum(b) / len(b)}

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            self.worker.reset_cache()
            self.ctrl.bcast({"flag": LoopFlag.STOP_LOOP})
        except Exception:
            pass
        for q in self._train_queues:
            q.put(None)
        for t in self._threads:         # daemon threads, but none may outlive the runtime
            if t is not threading.current_thread():
                t.join(timeout=5.0)
