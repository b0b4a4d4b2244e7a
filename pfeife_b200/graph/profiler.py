"""Graph bench: per-segment latency and memory of a captured graph on one device.

Behavioural counterpart of pfeife/local/graph_bench.py:172-625 and the three interpreters of
pfeife/graph/computation_graph.py:487-1450, folded into one node-by-node executor:
  * pass 1 runs the graph once with autograd on, recording per segment the growth of live
    memory (``act_mem``) and the transient peak (``temp_mem``) from allocator statistics, and
    keeps the model output for the caller;
  * pass 2 repeats the forward ``TIME_WARM_ITER + TIME_CHECK_ITER`` times with one CUDA event
    pair per segment (one device sync per iteration, none per segment);
  * pass 3 times whole forward vs forward+backward to get ``fb_ratio`` (clamped to >= 1);
  * optionally the optimizer step is timed on the real parameters and apportioned to segments
    by parameter bytes.
On CPU the same executor uses ``perf_counter`` and tensor sizes.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx

from ..utils import get_logger
from .capture import CapturedGraph
from . import comp_graph as comp_graph_mod
from .comp_graph import CompGraph, _tensor_leaves

TIME_WARM_ITER = 2
TIME_CHECK_ITER = 5
# a forward that replays as one CUDA graph in less than this share of its eagerly launched time
# was timed at the host's launch rate
HOST_BOUND_RATIO = 0.6


def gen_amp_context(device: torch.device, dtype: Optional[torch.dtype]):
    if dtype is None:
        return contextlib.nullcontext()
    return torch.autocast(device_type=device.type, dtype=dtype)


def _last_uses(gm: fx.GraphModule) -> Dict[str, List[str]]:
    """node name -> values that die right after it (freed by the executor)."""
    last: Dict[str, str] = {}
    for n in gm.graph.nodes:
        for a in n.all_input_nodes:
            last[a.name] = n.name
    out: Dict[str, List[str]] = {}
    for v, user in last.items():
        out.setdefault(user, []).append(v)
    return out


class SegmentExecutor:
    """Runs a captured graph node by node, calling ``on_segment_start/end`` at segment
    boundaries."""

    def __init__(self, graph: CompGraph):
        self.graph = graph
        self.gm = graph.captured.gm
        self.frees = _last_uses(self.gm)
        self.nodes = list(self.gm.graph.nodes)

    def run(self, args: Sequence[Any], on_start=None, on_end=None, keep_all: bool = False,
            on_value=None) -> Any:
        """``on_value(segment, value)`` sees every value a node produces (for hooks)."""
        env: Dict[str, Any] = {}
        it = iter(args)
        cur_seg = -1
        seg_of = self.graph.seg_of
        for n in self.nodes:
            if n.op == "placeholder":
                env[n.name] = next(it)
                continue
            if n.op == "output":
                if cur_seg >= 0 and on_end:
                    on_end(cur_seg)
                return fx.node.map_arg(n.args[0], lambda a: env[a.name])
            seg = seg_of[n.name]
            if seg != cur_seg:
                if cur_seg >= 0 and on_end:
                    on_end(cur_seg)
                if on_start:
                    on_start(seg)
                cur_seg = seg
            a = fx.node.map_arg(n.args, lambda x: env[x.name])
            k = fx.node.map_arg(n.kwargs, lambda x: env[x.name])
            if n.op == "call_function":
                env[n.name] = n.target(*a, **k)
            elif n.op == "call_method":
                env[n.name] = getattr(a[0], n.target)(*a[1:], **k)
            elif n.op == "call_module":
                env[n.name] = self.gm.get_submodule(n.target)(*a, **k)
            elif n.op == "get_attr":
                obj = self.gm
                for atom in n.target.split("."):
                    obj = getattr(obj, atom)
                env[n.name] = obj
            if on_value is not None and n.name in env:
                on_value(seg, env[n.name])
            if not keep_all:
                for v in self.frees.get(n.name, ()):
                    if v in env and self.gm.graph is not None:
                        del env[v]
        raise RuntimeError("graph has no output node")


def _graph_replay_ms(ex: "SegmentExecutor", args: Sequence[Any], amp, device) -> Optional[float]:
    """Device time of one forward of the whole graph replayed as a CUDA graph (mean of
    ``TIME_CHECK_ITER`` replays), or None when the forward cannot be captured."""
    try:
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.no_grad(), amp():
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                ex.run(args)
        for _ in range(TIME_WARM_ITER):
            g.replay()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(TIME_CHECK_ITER):
            g.replay()
        e.record()
        torch.cuda.synchronize(device)
        ms = s.elapsed_time(e) / TIME_CHECK_ITER
        del g
        return ms
    except Exception as exc:     # an op that cannot be captured: keep the eager figures
        get_logger().info("forward not captured as one graph (%s: %s)", type(exc).__name__,
                          str(exc).splitlines()[0] if str(exc) else "")
        try:
            torch.cuda.synchronize(device)
        except Exception:
            pass
        return None


def _kernel_busy_ms(ex: "SegmentExecutor", args: Sequence[Any], amp, device
                    ) -> Optional[Tuple[float, float]]:
    """Sums of the kernel durations (ms) of one forward and of one backward (activity records of
    the profiler: launch gaps do not count), or None when no records could be had."""
    try:
        from torch.profiler import ProfilerActivity, profile

        def busy(fn):
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                r = fn()
                torch.cuda.synchronize(device)
            return r, sum(float(getattr(ev, "device_time_total", 0) or 0) for ev in prof.events())

        def fwd():
            with amp():
                return ex.run(args)

        out, f_us = busy(fwd)
        loss = _sum_outputs(out)
        if loss is None or f_us <= 0:
            return None
        _, b_us = busy(loss.backward)
        return (f_us / 1e3, b_us / 1e3) if b_us > 0 else None
    except Exception as exc:
        get_logger().info("no kernel activity records (%s)", type(exc).__name__)
        return None


def segment_backward_times(ex: "SegmentExecutor", args: Sequence[Any], amp, device,
                           total_ms: float) -> Optional[List[float]]:
    """Backward time of every segment, from one eager backward: a gradient hook on every value a
    segment produces stamps the moment that value's gradient is complete; the latest stamp of a
    segment is when the backward reaches it, and a segment's backward lasts until the backward
    reaches the segment before it.  Only the proportions are kept: the list is scaled to sum to
    ``total_ms`` (the backward total the planner already uses), so an eager pass that ran at the
    host's launch rate still cannot change the predicted step, only how it is split.

    (The reference applies one backward/forward ratio to every segment,
    pfeife/local/graph_bench.py; attention, GEMM and norm segments differ by a factor of two.)"""
    is_cuda = device.type == "cuda"
    n_seg = len(ex.graph.nodes)
    stamps: Dict[int, list] = {}

    def now():
        if is_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    def attach(seg, value):
        for t in _tensor_leaves(value):
            if torch.is_tensor(t) and t.requires_grad and t.dtype.is_floating_point:
                t.register_hook(lambda g, s=seg: stamps.setdefault(s, []).append(now()))

    try:
        with amp():
            out = ex.run(args, on_value=attach)
        loss = _sum_outputs(out)
        if loss is None:
            return None
        if is_cuda:
            torch.cuda.synchronize(device)
        begin = now()
        loss.backward()
        end = now()
        if is_cuda:
            torch.cuda.synchronize(device)
        at = (lambda x: begin.elapsed_time(x)) if is_cuda else (lambda x: (x - begin) * 1e3)
        reached = [max((at(x) for x in stamps[k]), default=None) if k in stamps else None
                   for k in range(n_seg)]
        # a segment without a differentiable value of its own is reached when the next one is
        nxt = 0.0
        for k in range(n_seg - 1, -1, -1):
            if reached[k] is None:
                reached[k] = nxt
            nxt = reached[k]
        times = []
        for k in range(n_seg):
            until = at(end) if k == 0 else reached[k - 1]
            times.append(max(0.0, until - reached[k]))
        total = sum(times)
        if total <= 0.0:
            return None
        return [t * total_ms / total for t in times]
    except Exception as exc:
        get_logger().info("per-segment backward timing unavailable (%s: %s)",
                          type(exc).__name__, str(exc).splitlines()[0] if str(exc) else "")
        return None


def _sum_outputs(out: Any) -> Optional[torch.Tensor]:
    total = None
    for t in _tensor_leaves(out if not isinstance(out, dict) else list(out.values())):
        if t.dtype.is_floating_point and t.requires_grad:
            s = t.float().sum()
            total = s if total is None else total + s
    return total


def measure_optimizer(graph: CompGraph, option, device: torch.device) -> float:
    """Times ``TIME_CHECK_ITER`` optimizer steps on copies of the graph's parameters (gradients
    set to zeros) and apportions the mean to segments by parameter bytes.  Returns the mean in ms."""
    params = [i.tensor for i in graph.captured.params if i.tensor.requires_grad]
    if not params:
        return 0.0
    # the steps run on stand-ins of the same shapes: the real parameters are saved for the
    # backward of the probing call that is still in flight and must keep their versions
    standins = [torch.nn.Parameter(p.detach().clone()) for p in params]
    for q in standins:
        q.grad = torch.zeros_like(q)
    opt = option.make_optimizer(standins)
    sync = torch.cuda.synchronize if device.type == "cuda" else (lambda: None)
    for _ in range(TIME_WARM_ITER):
        opt.step()
    sync()
    t0 = time.perf_counter()
    for _ in range(TIME_CHECK_ITER):
        opt.step()
    sync()
    ms = (time.perf_counter() - t0) * 1e3 / TIME_CHECK_ITER
    del opt, standins
    total = sum(n.param_bytes for n in graph.nodes) or 1
    for n in graph.nodes:
        n.optim_time = ms * n.param_bytes / total
    return ms


def gen_local_comp_graph(captured: CapturedGraph, args: Sequence[Any], device: torch.device,
                         option) -> Tuple[CompGraph, Any]:
    """Profiles `captured` with call arguments `args` (placeholder order) on `device`.

    Returns the profiled graph and the output of one real forward (so the probing call of the
    user's ``exec_fn`` can continue into its loss and backward)."""
    log = get_logger()
    graph = CompGraph(captured)
    ex = SegmentExecutor(graph)
    is_cuda = device.type == "cuda"
    amp = lambda: gen_amp_context(device, option.mixed_precision)

    cached = option.graph_bench and os.path.exists(option.graph_bench)
    # ---- pass 1: one real forward with memory statistics.  It keeps every activation alive
    #      (the caller's loss and backward continue from its output), so a model whose
    #      activations outgrow the device is profiled with its saved tensors parked in pinned
    #      host memory from the segment on at which reserved memory passes GRAPH_FETCH_MEM_CAP
    #      of the device (pfeife/graph/computation_graph.py:926-963 offloads the same way);
    #      the segments after that point keep their analytic activation sizes.
    mem_before: Dict[int, int] = {}
    offload = contextlib.ExitStack()
    offloaded_from = [None]
    if is_cuda:
        torch.cuda.synchronize(device)
        total_mem = torch.cuda.get_device_properties(device).total_memory

        def on_start(seg):
            torch.cuda.reset_peak_memory_stats(device)
            mem_before[seg] = torch.cuda.memory_allocated(device)

        def on_end(seg):
            now = torch.cuda.memory_allocated(device)
            peak = torch.cuda.max_memory_allocated(device)
            node = graph.nodes[seg]
            if offloaded_from[0] is None:
                node.act_mem = max(0, now - mem_before[seg])
                node.temp_mem = max(node.act_mem, peak - mem_before[seg])
                if torch.cuda.memory_reserved(device) > comp_graph_mod.GRAPH_FETCH_MEM_CAP * total_mem:
                    offloaded_from[0] = seg + 1
                    offload.enter_context(torch.autograd.graph.save_on_cpu(pin_memory=True))
                    log.info("profiling pass: activations go to host memory from segment %d on",
                             seg + 1)
            else:
                node.temp_mem = max(node.act_mem, peak - mem_before[seg])
    else:
        on_start = on_end = None
    with offload, amp():
        output = ex.run(args, None if cached else on_start, None if cached else on_end)
    if cached:
        graph.load_graph_data(option.graph_bench)
        log.info("loaded graph bench from %s: %s", option.graph_bench, graph.summary())
        return graph, output
    # the segment order the planner cuts (--linearizer): chosen from the memory figures of pass
    # 1, before the timing passes run in that order (pfeife/local/graph_bench.py:436-438)
    if graph.linearize(getattr(option, "linearizer", "none")):
        ex = SegmentExecutor(graph)
        log.info("segments re-ordered by the %s linearizer", option.linearizer)

    # ---- pass 2: per-segment forward timing
    graph_fwd_ms = None
    n_seg = len(graph.nodes)
    acc = [0.0] * n_seg
    for it in range(TIME_WARM_ITER + TIME_CHECK_ITER):
        timed = it >= TIME_WARM_ITER
        if is_cuda:
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_seg)]
            ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_seg)]
            with torch.no_grad(), amp():
                ex.run(args, lambda s: starts[s].record(), lambda s: ends[s].record())
            torch.cuda.synchronize(device)
            if timed:
                for s in range(n_seg):
                    acc[s] += starts[s].elapsed_time(ends[s])
        else:
            t: Dict[int, float] = {}
            with torch.no_grad(), amp():
                ex.run(args, lambda s: t.__setitem__(s, time.perf_counter()),
                       lambda s: acc.__setitem__(s, acc[s] + (time.perf_counter() - t[s]) * 1e3
                                                 if timed else acc[s]))
    for s in range(n_seg):
        graph.nodes[s].comp_time = max(acc[s] / TIME_CHECK_ITER, 1e-4)
    host_bound = False
    if is_cuda and getattr(option, "cuda_graphs", False):
        # The run replays CUDA graphs, the pass above launched eagerly: with kernels of a few
        # microseconds it measured the host's launch rate, not the device.  The whole forward
        # replayed as one graph gives the device time.  Where the host clearly bounds the eager
        # pass (the replay takes less than HOST_BOUND_RATIO of it) the segment times keep their
        # proportions and are scaled to the replay.  Above that ratio the eager figures stay:
        # with the wall-clock backward/forward ratio of pass 3 they predicted the replayed step
        # of ViT-g/14 within 3 % (1 and 2 GPUs, data- and pipeline-parallel), whereas the
        # corrected pair under-predicted it by 11 %.
        replay = _graph_replay_ms(ex, args, amp, device)
        eager = sum(n.comp_time for n in graph.nodes)
        if replay is not None and 0.0 < replay < eager:
            k = replay / eager
            host_bound = k < HOST_BOUND_RATIO
            if host_bound:
                graph_fwd_ms = replay
                for n in graph.nodes:
                    n.comp_time = max(n.comp_time * k, 1e-4)
            log.info("forward as one CUDA graph: %.3f ms against %.3f ms launched eagerly%s",
                     replay, eager, f"; segment times scaled by {k:.3f}" if host_bound else "")

    # ---- pass 3: forward vs backward wall clock
    sync = (lambda: torch.cuda.synchronize(device)) if is_cuda else (lambda: None)
    fwd_ms = bwd_ms = 0.0
    for it in range(TIME_WARM_ITER + TIME_CHECK_ITER):
        sync()
        t0 = time.perf_counter()
        with amp():
            out = ex.run(args)
        loss = _sum_outputs(out)
        sync()
        t1 = time.perf_counter()
        if loss is not None:
            loss.backward()
        sync()
        t2 = time.perf_counter()
        if it >= TIME_WARM_ITER:
            fwd_ms += (t1 - t0) * 1e3
            bwd_ms += (t2 - t1) * 1e3
    graph.fb_ratio = max(1.0, bwd_ms / fwd_ms) if fwd_ms > 0 else 2.0
    if host_bound:
        # under graph replay the ratio is one of device times; the wall clock above is the
        # host's launch rate in both directions when the kernels are short
        busy = _kernel_busy_ms(ex, args, amp, device)
        if busy is not None:
            # Two bounds.  The wall-clock ratio is too low when both directions ran at the host's
            # launch rate.  The backward's kernel time against the forward as it replays is too
            # high: this probing backward still writes every parameter gradient to a tensor of
            # its own and lets autograd accumulate it, where the stages add into the gradient
            # bucket from the GEMM epilogue.  The geometric mean of the two is used.
            f_ms, b_ms = busy
            upper = b_ms / graph_fwd_ms if graph_fwd_ms else b_ms / f_ms
            ratio = (max(graph.fb_ratio, 1.0) * max(upper, 1.0)) ** 0.5
            log.info("backward / forward: %.3f (wall clock %.3f, device time %.3f; kernels "
                     "%.3f / %.3f ms)", ratio, graph.fb_ratio, upper, b_ms, f_ms)
            graph.fb_ratio = max(1.0, ratio)
    # per-segment backward times (proportions of one more eager backward, total unchanged)
    back = segment_backward_times(ex, args, amp, device,
                                  graph.fb_ratio * sum(n.comp_time for n in graph.nodes))
    if back is not None:
        for n, b in zip(graph.nodes, back):
            n.back_time = max(b, 1e-4)
    for i in captured.params:
        i.tensor.grad = None
    log.info("forward: %.4f ms, backward: %.4f ms", fwd_ms / TIME_CHECK_ITER,
             bwd_ms / TIME_CHECK_ITER)

    if not option.no_bench_optimizer:
        measure_optimizer(graph, option, device)
    if option.graph_bench:
        graph.save_graph_data(option.graph_bench)
    return graph, output


def run_unprofiled(captured: CapturedGraph, args: Sequence[Any], device: torch.device, option
                   ) -> Tuple[CompGraph, Any]:
    """The segmented graph and the output of one forward, without measuring anything: for a
    rank that receives the statistics from the rank that profiled."""
    graph = CompGraph(captured)
    with gen_amp_context(device, option.mixed_precision):
        output = SegmentExecutor(graph).run(args)
    return graph, output


def gen_comp_graph_cpu(captured: CapturedGraph, args: Sequence[Any], option
                       ) -> Tuple[CompGraph, Any]:
    """Unit-time profile for CPU tests: every segment costs 1 ms forward, ``fb_ratio`` 2
    (pfeife/local/graph_bench.py:125-144)."""
    graph = CompGraph(captured)
    with gen_amp_context(torch.device("cpu"), option.mixed_precision):
        output = SegmentExecutor(graph).run(args)
    graph.linearize(getattr(option, "linearizer", "none"))
    for n in graph.nodes:
        n.comp_time = 1.0
    graph.fb_ratio = 2.0
    return graph, output
