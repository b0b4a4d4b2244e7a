"""Stage executor: runs one rank's step program (receive, forward, send, receive-grad,
backward, send-grad, optimizer) over its pipeline stages.

Role of pfeife/mp/worker.py:148-1590 (``ProcessWorker``) with a different communication
design:
  * control plane on the host (gloo object broadcast: options, plans, per-step flags and
    optimizer hyper-parameters) instead of pickles through NCCL byte tensors;
  * data plane = FIFO directed channels (see transport.py).  The order of messages on a channel
    is derived from the sender's step program, so receives are posted ahead of need, into
    persistent per-(edge, micro-batch) buffers, with a configurable look-ahead, and no global
    transfer order has to be simulated to stay deadlock-free;
  * parameters live in flat buffers (params.py); the gradient of a parameter shared by stages
    on several ranks is summed over those ranks before the optimizer step
    (pfeife/mp/worker.py:316-408);
  * one global loss scale with a PPxDP-wide non-finite flag (the reference lets every worker
    scale independently).
The same class serves the process-per-GPU runtime (``DistTransport``) and the single-process
thread-per-device runtime (``LocalTransport``).
"""
from __future__ import annotations

import contextlib
import enum
import os
import threading
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..graph.partition import OUTSIDE, PartitionGraph, StageSpec
from ..graph.profiler import gen_amp_context
from ..parallel.schedule import Step, StepWork
from ..utils import fmem, get_logger
from ..utils.timing import CPUTimeRecorder, CUDATimeRecorder
from .params import LossScaler, RankParams, StateEntry
from .transport import Handle, Transport


class LoopFlag(enum.IntEnum):
    STOP_LOOP = 0
    CONTINUE_LOOP = 1
    GATHER_PARAMS = 2
    LOG_MEMORY_USAGE = 3
    LOAD_PARAMS = 4
    EVAL_LOOP = 5
    REPORT_TIMES = 6


# message key: (is_grad, producer_stage, producer_output, consumer_stage, consumer_input, mb)
MsgKey = Tuple[bool, int, int, int, int, int]


@dataclass
class _Msg:
    key: MsgKey
    src_rank: int
    dst_rank: int
    meta: Any                      # ShapeMeta


class CommPlan:
    """Static message bookkeeping of one rank for one plan: which messages each step sends or
    needs, and the FIFO order of every channel this rank takes part in."""

    def __init__(self, part: PartitionGraph, steps_by_rank: List[List[Step]], batch_cnt: int,
                 rank: int, main_rank: int, training: bool = True):
        self.part, self.rank, self.main_rank, self.batch_cnt = part, rank, main_rank, batch_cnt
        stages = part.stages
        rank_of = lambda s: main_rank if s == OUTSIDE else stages[s].rank
        self.send_at: Dict[Tuple[int, int, int], List[_Msg]] = {}    # (work, stage, mb) -> msgs
        self.need_at: Dict[Tuple[int, int, int], List[_Msg]] = {}
        self.input_msgs: List[_Msg] = []          # user inputs leaving the main rank, issue order
        self.channel_send: Dict[int, List[_Msg]] = {}   # dst rank -> FIFO of my sends
        self.channel_recv: Dict[int, List[_Msg]] = {}   # src rank -> FIFO of my receives
        self.channels: List[Tuple[int, int]] = []

        # FIFO order of every channel = walk every sender's program
        fifo: Dict[Tuple[int, int], List[_Msg]] = {}

        def emit(msg: _Msg):
            if msg.src_rank == msg.dst_rank:
                return
            fifo.setdefault((msg.src_rank, msg.dst_rank), []).append(msg)

        # user inputs: issued by the main rank before its first step, micro-batch major
        for mb in range(batch_cnt):
            for sp in stages:
                for j, inp in enumerate(sp.inputs):
                    if inp.kind == "input" and inp.meta is not None:
                        m = _Msg((False, OUTSIDE, inp.ph_index, sp.idx, j, mb), main_rank,
                                 sp.rank, inp.meta)
                        if sp.rank != main_rank:
                            emit(m)
                            if rank == main_rank:
                                self.input_msgs.append(m)
                        if sp.rank == rank and sp.rank != main_rank:
                            self.need_at.setdefault((int(StepWork.RECV_ACT), sp.idx, mb),
                                                    []).append(m)
        for r, steps in enumerate(steps_by_rank):
            for st in steps:
                if st.work == StepWork.SEND_ACT:
                    sp = stages[st.node_id]
                    for j, out in enumerate(sp.outputs):
                        for (c, cin) in out.consumers:
                            if c == OUTSIDE:
                                continue
                            m = _Msg((False, sp.idx, j, c, cin, st.batch_id), sp.rank,
                                     rank_of(c), out.meta)
                            emit(m)
                            if r == rank:
                                self.send_at.setdefault((int(StepWork.SEND_ACT), sp.idx,
                                                         st.batch_id), []).append(m)
                            if rank_of(c) == rank:
                                self.need_at.setdefault((int(StepWork.RECV_ACT), c, st.batch_id),
                                                        []).append(m)
                elif st.work == StepWork.SEND_GRAD and training:
                    sp = stages[st.node_id]
                    for j, inp in enumerate(sp.inputs):
                        if inp.kind != "edge" or inp.meta is None or not inp.meta.requires_grad:
                            continue
                        m = _Msg((True, inp.src_stage, inp.src_output, sp.idx, j, st.batch_id),
                                 sp.rank, rank_of(inp.src_stage), inp.meta)
                        emit(m)
                        if r == rank:
                            self.send_at.setdefault((int(StepWork.SEND_GRAD), sp.idx,
                                                     st.batch_id), []).append(m)
                        if rank_of(inp.src_stage) == rank:
                            self.need_at.setdefault((int(StepWork.RECV_GRAD), inp.src_stage,
                                                     st.batch_id), []).append(m)
        self.recv_pos: Dict[int, Dict[MsgKey, int]] = {}   # src rank -> message key -> position
        for (a, b), msgs in fifo.items():
            self.channels.append((a, b))
            if a == rank:
                self.channel_send[b] = msgs
            if b == rank:
                self.channel_recv[a] = msgs
                self.recv_pos[a] = {m.key: i for i, m in enumerate(msgs)}


def _lib_add(n: int) -> None:
    from ..ops import _lib
    _lib.add_launches(n)


class _GraphedStage:
    """CUDA graphs of one stage's forward and backward for one in-flight slot.

    The forward graph reads ``static_ins`` and produces ``static_outs``; its saved activations
    live in the graph's private memory pool until the backward graph of the same slot has been
    replayed.  The backward graph reads ``static_gouts``, accumulates parameter gradients in
    place (bucket views / wgrad epilogues) and leaves the gradients of the stage inputs in
    ``static_ins[j].grad``."""

    def __init__(self):
        self.fwd = None
        self.bwd = None
        self.static_ins: List[Any] = []
        self.static_outs: Tuple[Any, ...] = ()
        self.grad_outs: List[Tuple[int, torch.Tensor]] = []   # (output index, static grad)
        self.failed = False
        self.fwd_kernels = 0     # native kernels recorded in each graph (for launch accounting)
        self.bwd_kernels = 0


def inflight_slots(steps: Sequence[Step]) -> Tuple[Dict[Tuple[int, int], int], int]:
    """(stage, micro-batch) -> slot such that two micro-batches of a stage share a slot only
    when the first one's backward precedes the second one's forward."""
    free: Dict[int, List[int]] = {}
    nxt: Dict[int, int] = {}
    slot: Dict[Tuple[int, int], int] = {}
    for st in steps:
        if st.work == StepWork.FORWARD:
            fl = free.setdefault(st.node_id, [])
            if fl:
                slot[(st.node_id, st.batch_id)] = fl.pop(0)
            else:
                slot[(st.node_id, st.batch_id)] = nxt.get(st.node_id, 0)
                nxt[st.node_id] = nxt.get(st.node_id, 0) + 1
        elif st.work == StepWork.BACKWARD:
            free.setdefault(st.node_id, []).append(slot[(st.node_id, st.batch_id)])
            free[st.node_id].sort()
    return slot, max(nxt.values(), default=0)


class StageWorker:
    """Executes the step program of one pipeline rank."""

    def __init__(self, pp_rank: int, pp_size: int, device: torch.device, option,
                 transport: Optional[Transport], runner=None, global_ranks: Optional[List[int]] = None):
        self.pp_rank, self.pp_size, self.device, self.option = pp_rank, pp_size, device, option
        self.transport = transport
        self.runner = runner              # main rank only: delivers outputs / receives loss grads
        self.global_ranks = global_ranks or list(range(pp_size))   # pp rank -> global rank
        self.main_rank = pp_size - 1
        self.is_main = pp_rank == self.main_rank
        self.log = get_logger()
        self.part: Optional[PartitionGraph] = None
        self.params: Optional[RankParams] = None
        self.steps: List[Step] = []
        self.eval_steps: List[Step] = []
        self.comm: Optional[CommPlan] = None
        self.batch_cnt = option.batch_cnt
        self.scaler = LossScaler(device, option.mixed_precision == torch.float16,
                                 option.init_loss_scale)
        self.recorder = CUDATimeRecorder() if device.type == "cuda" else CPUTimeRecorder()
        self.recv_lookahead = 2
        self.dp = None                     # data-parallel reducer (set by the runtime front-end)
        self.shared_groups: Dict[Tuple[int, ...], Any] = {}
        self.idle_mem = 0
        self.use_graphs = bool(getattr(option, "cuda_graphs", False)) and device.type == "cuda"
        self.graph_warmup_steps = 1       # eager steps before capture (lazy inits, autotune)
        self.graphs: Dict[Tuple[int, int, int], _GraphedStage] = {}
        self.slot_of: Dict[Tuple[int, int], int] = {}
        self.graph_key: Dict[Tuple[int, int], Tuple[int, int, int]] = {}
        self._example_ins: Dict[int, List[Any]] = {}     # stage -> inputs of an eager forward
        self._captured_upfront = False
        # stages whose row-sharded weights were completed since the last optimizer step
        self.gathered_stages: set = set()
        # True when the job has more ranks than this stage's replicas (set by the front-end)
        self.inf_sync_job_wide = pp_size > 1
        self.train_steps_done = 0
        self.opt_event_log: List[Tuple[Any, Any]] = []
        self._reset_step_state()

    # ------------------------------------------------------------------ plan installation
    def set_partition_graph(self, part: PartitionGraph, entries: Sequence[StateEntry],
                            optimizer_type: str, hyper: List[Dict[str, Any]]) -> None:
        self.part = part
        lp = self.option.mixed_precision
        alloc = self.dp.allocator() if (self.dp is not None and hasattr(self.dp, "allocator")) \
            else None
        # --use_fsdp with the fused data-parallel step: weight matrices stay row-sharded after
        # the optimizer step and are gathered by the first GEMM that reads them
        defer = bool(getattr(self.option, "use_fsdp", False)) and self.dp is not None and \
            getattr(self.dp, "fused", False)
        self.params = RankParams(entries, self.device, lp, optimizer_type, hyper, alloc=alloc,
                                 defer_gather=defer)
        self.stage_mods: Dict[int, Any] = {}
        for sp in part.stages_of_rank(self.pp_rank):
            gm = sp.gm
            gm.to(self.device)
            if self.option.compiler:
                from ..compile import compile_module
                gm = compile_module(self.option.compiler, gm)
            self.stage_mods[sp.idx] = gm
        if self.dp is not None:
            self.dp.attach(self.params)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            self.idle_mem = torch.cuda.memory_allocated(self.device)

    def set_scheduler_steps(self, steps_by_rank: List[List[Step]],
                            eval_steps_by_rank: Optional[List[List[Step]]] = None) -> None:
        self.steps = list(steps_by_rank[self.pp_rank])
        self.comm = CommPlan(self.part, steps_by_rank, self.batch_cnt, self.pp_rank,
                             self.main_rank)
        if eval_steps_by_rank is not None:
            self.eval_steps = list(eval_steps_by_rank[self.pp_rank])
            self.eval_comm = CommPlan(self.part, eval_steps_by_rank, self.batch_cnt,
                                      self.pp_rank, self.main_rank, training=False)
        self.recv_bufs: Dict[MsgKey, torch.Tensor] = {}
        self.zero_bufs: Dict[MsgKey, torch.Tensor] = {}
        self.slot_of, _ = inflight_slots(self.steps)
        # the orderings the buffers of this rank rely on (cheap: one pass over the program)
        from .hazards import program_hazards
        problems = program_hazards(self.steps, self.slot_of)
        if problems:
            raise RuntimeError("step program of pipeline rank %d is unsafe: %s"
                               % (self.pp_rank, "; ".join(problems[:5])))
        if self.transport is not None:
            g = self.global_ranks
            self.transport.warm_up([(g[a], g[b]) for a, b in self.comm.channels])

    def _buf(self, msg: _Msg) -> torch.Tensor:
        b = self.recv_bufs.get(msg.key)
        if b is None:
            b = torch.empty(msg.meta.size, dtype=msg.meta.dtype, device=self.device)
            self.recv_bufs[msg.key] = b
        return b

    # ------------------------------------------------------------------ per-step state
    def _reset_step_state(self) -> None:
        self.sends: List[Handle] = []
        self.send_of: Dict[int, Handle] = {}       # source address -> its latest send
        self.recv_handles: Dict[MsgKey, Handle] = {}
        self.recv_cursor: Dict[int, int] = {}
        self.local_vals: Dict[MsgKey, torch.Tensor] = {}       # same-rank hand-offs
        self.fw_inputs: Dict[Tuple[int, int], List[Any]] = {}
        self.fw_outputs: Dict[Tuple[int, int], Tuple[Any, ...]] = {}
        self.user_inputs: Dict[int, Dict[int, Any]] = {}       # mb -> {ph_index: value}
        self.loss_grads: Dict[int, Dict[int, Optional[torch.Tensor]]] = {}
        self.bw_events: Dict[int, threading.Event] = {}

    def reset_cache(self) -> None:
        for h in self.sends:
            h.wait()
        self._reset_step_state()
        if getattr(self.option, "no_io_cache", False) and hasattr(self, "recv_bufs"):
            # --no_io_cache: receive buffers live for one step instead of being kept per
            # (edge, micro-batch) for the whole run (pfeife/local/worker.py:403-420)
            self.recv_bufs.clear()
            self.zero_bufs.clear()

    # ------------------------------------------------------------------ receive machinery
    def _post_until(self, comm: CommPlan, src: int, msg: _Msg) -> None:
        """Posts the receives of channel src->me in FIFO order up to `msg` plus look-ahead."""
        fifo = comm.channel_recv[src]
        cur = self.recv_cursor.get(src, 0)
        want = comm.recv_pos[src].get(msg.key)
        assert want is not None, f"message {msg.key} not on channel {src}->{self.pp_rank}"
        upto = min(len(fifo), max(cur, want + 1 + self.recv_lookahead))
        g = self.global_ranks
        for i in range(cur, upto):
            m = fifo[i]
            self.recv_handles[m.key] = self.transport.irecv(self._buf(m), g[src])
        self.recv_cursor[src] = max(cur, upto)

    def _receive(self, comm: CommPlan, msgs: Sequence[_Msg]) -> None:
        for m in msgs:
            if m.src_rank == m.dst_rank:
                continue
            if m.key not in self.recv_handles:
                self._post_until(comm, m.src_rank, m)
        for m in msgs:
            if m.src_rank != m.dst_rank:
                self.recv_handles[m.key].wait()

    def _send(self, msg: _Msg, tensor: torch.Tensor) -> None:
        if msg.src_rank == msg.dst_rank:
            self.local_vals[msg.key] = tensor
            return
        t = tensor.detach()
        if not t.is_contiguous():
            t = t.contiguous()
        if t.dtype != msg.meta.dtype:
            t = t.to(msg.meta.dtype)
        h = self.transport.isend(t, self.global_ranks[msg.dst_rank])
        self.sends.append(h)
        self.send_of[t.data_ptr()] = h      # see _wait_sends_from

    def _wait_sends_from(self, tensors) -> None:
        """Before a graph replay overwrites its static buffers: the stream waits for the
        transfers that still read them (a send is only posted when it is issued; the peer may
        match it much later)."""
        for t in tensors:
            if torch.is_tensor(t):
                h = self.send_of.pop(t.data_ptr(), None)
                if h is not None:
                    h.wait()

    def _take(self, msg: _Msg) -> torch.Tensor:
        if msg.src_rank == msg.dst_rank:
            return self.local_vals.pop(msg.key)
        return self.recv_bufs[msg.key]

    # ------------------------------------------------------------------ main-rank hooks
    def submit_inputs(self, mb: int, values: Dict[int, Any]) -> None:
        self.user_inputs[mb] = values
        self.loss_grads[mb] = {}
        self.bw_events[mb] = threading.Event()

    def distribute_inputs(self, comm: CommPlan) -> None:
        """Main rank: sends every micro-batch's user inputs to the ranks whose stages read them
        (pfeife/mp/worker.py:818-840)."""
        for m in comm.input_msgs:
            _, _, ph, _, _, mb = m.key
            v = self.user_inputs[mb][ph]
            self._send(m, v.to(self.device) if v.device != self.device else v)

    def recv_loss_grad(self, mb: int, out_idx: int, grad: Optional[torch.Tensor]) -> None:
        self.loss_grads[mb][out_idx] = grad

    def loss_backward_done(self, mb: int) -> None:
        ev = self.bw_events.get(mb)
        if ev is not None:
            ev.set()

    # ------------------------------------------------------------------ step handlers
    def _stage_inputs(self, comm: CommPlan, sp: StageSpec, mb: int) -> List[Any]:
        need = {m.key[4]: m for m in comm.need_at.get((int(StepWork.RECV_ACT), sp.idx, mb), [])}
        ins: List[Any] = []
        for j, inp in enumerate(sp.inputs):
            if inp.kind == "state":
                ins.append(self.params.tensor_for(inp.ph_index))
            elif inp.kind == "input":
                if self.is_main:
                    v = self.user_inputs[mb][inp.ph_index]
                    if torch.is_tensor(v) and v.device != self.device:
                        v = v.to(self.device, non_blocking=True)
                    ins.append(v)
                elif j in need:
                    ins.append(self._take(need[j]))
                else:
                    raise RuntimeError(f"stage {sp.idx} input {inp.name} is not a tensor and "
                                       "cannot be shipped to a worker rank")
            else:
                t = self._take(need[j]).detach()
                if inp.meta is not None and inp.meta.requires_grad and torch.is_grad_enabled():
                    t.requires_grad_(True)
                ins.append(t)
        return ins

    def forward(self, comm: CommPlan, stage: int, mb: int) -> None:
        sp = self.part.stages[stage]
        ins = self._stage_inputs(comm, sp, mb)
        start = self.recorder.record_event(self.device)
        # the first forward of a stage after an optimizer step completes its row-sharded weights
        # (deferred all-gather); it is a graph of its own, since later forwards must not gather
        gather = self._defers_gather() and stage not in self.gathered_stages
        self.gathered_stages.add(stage)
        if self.use_graphs and torch.is_grad_enabled() and \
                self.train_steps_done >= self.graph_warmup_steps:
            gs = self._graph_for(sp, stage, mb, ins, int(gather))
            if gs is not None:
                with torch.no_grad():       # the static inputs are leaves that require grad
                    for dst, src in zip(gs.static_ins, ins):
                        if dst is not src and torch.is_tensor(dst):
                            dst.copy_(src, non_blocking=True)
                self._wait_sends_from(gs.static_outs)
                gs.fwd.replay()
                _lib_add(gs.fwd_kernels)
                self.recorder.append_fw(stage, start, self.recorder.record_event(self.device))
                self.fw_inputs[(stage, mb)] = gs.static_ins
                self.fw_outputs[(stage, mb)] = gs.static_outs
                return
        self.graph_key.pop((stage, mb), None)
        if self.use_graphs and torch.is_grad_enabled() and stage not in self._example_ins:
            self._example_ins[stage] = list(ins)     # shapes / dtypes for the capture phase
        if gather:
            from ..ops import functional as Fn
            Fn.gather_session(True)
        try:
            with gen_amp_context(self.device, self.option.mixed_precision):
                outs = self.stage_mods[stage](*ins)
        finally:
            if gather:
                Fn.gather_session(False)
        self.recorder.append_fw(stage, start, self.recorder.record_event(self.device))
        if not isinstance(outs, (tuple, list)):
            outs = (outs,)
        self.fw_inputs[(stage, mb)] = ins
        self.fw_outputs[(stage, mb)] = tuple(outs)

    # ------------------------------------------------------------------ CUDA graphs
    def _defers_gather(self) -> bool:
        return bool(getattr(self.dp, "deferred_below", None)) and getattr(self.dp, "fused", False)

    def _graph_for(self, sp: StageSpec, stage: int, mb: int, ins: List[Any], gather: int = 0
                   ) -> Optional[_GraphedStage]:
        key = (stage, self.slot_of.get((stage, mb), 0), gather)
        self.graph_key[(stage, mb)] = key
        gs = self.graphs.get(key)
        if gs is not None:
            return None if gs.failed else gs
        gs = _GraphedStage()
        self.graphs[key] = gs
        # A capture can break on work that only happens the first time a process does it (a
        # library handle or a kernel image created lazily inside the captured region): the
        # broken attempt has then done that work, and a second attempt on a fresh memory pool
        # goes through.  Only when that fails too does the stage stay on the eager path.
        for attempt in (0, 1):
            try:
                if gather:
                    from ..ops import functional as Fn
                    Fn.gather_session(True)
                try:
                    self._capture(gs, sp, stage, ins)
                finally:
                    if gather:
                        Fn.gather_session(False)
                return gs
            except Exception as e:
                import traceback
                where = " <- ".join(f"{f.name}:{f.lineno}" for f in
                                    reversed(traceback.extract_tb(e.__traceback__)[-4:]))
                cause = e.__context__
                if cause is not None and cause.__traceback__ is not None:
                    where += " [first error at " + " <- ".join(
                        f"{f.name}:{f.lineno}" for f in
                        reversed(traceback.extract_tb(cause.__traceback__)[-6:])) + "]"
                self.log.log(20 if attempt == 0 else 30,
                             "CUDA graph capture of stage %d failed (%s: %s) at %s%s; %s", stage,
                             type(e).__name__, str(e).splitlines()[0], where,
                             f" after {type(cause).__name__}: {str(cause).splitlines()[0]}"
                             if cause is not None else "",
                             "trying once more" if attempt == 0 else "running it eagerly")
                # (a capture that broke leaves its memory pool marked as recording: the next
                # attempt makes a pool of its own)
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
        gs.failed = True
        return None

    def capture_all(self) -> None:
        """Captures the graphs of every (stage, in-flight slot) of this rank's step program in
        one go, between two steps, from the inputs an eager step left behind.  Nothing of the
        step is in flight then: no transfer is posted, no front-end thread computes, and a
        capture's device-wide synchronisation cannot wait for a peer.  (Capturing lazily inside
        the step works for a single stage per job; with stage hand-offs in flight captures were
        invalidated.)"""
        self._captured_upfront = True
        defers = self._defers_gather()
        seen_stage: set = set()
        for st in self.steps:
            if st.work != StepWork.FORWARD:
                continue
            stage, mb = st.node_id, st.batch_id
            ins = self._example_ins.get(stage)
            if ins is None:
                continue
            gather = int(defers and stage not in seen_stage)
            seen_stage.add(stage)
            key = (stage, self.slot_of.get((stage, mb), 0), gather)
            if key in self.graphs:
                continue
            self._graph_for(self.part.stages[stage], stage, mb, ins, gather)
        self.graph_key.clear()

    def _capture(self, gs: _GraphedStage, sp: StageSpec, stage: int, ins: List[Any]) -> None:
        # One memory pool per (stage, slot): its forward and backward graphs always replay in the
        # order they were captured.  Graphs of different slots replay interleaved (forward of
        # slot 1 between forward and backward of slot 0); in a shared pool the later capture
        # would have been handed the blocks that the earlier backward capture freed -- the
        # activations slot 0's forward saves for its backward -- and overwrite them on replay.
        pool = torch.cuda.graph_pool_handle()
        static_ins: List[Any] = []
        for inp, v in zip(sp.inputs, ins):
            if inp.kind == "state" or not torch.is_tensor(v):
                static_ins.append(v)
                continue
            # a fresh leaf: copying from a tensor that requires grad with autograd recording
            # would hang a CopyBackwards node (made outside the capture, on the stream that is
            # current here) under the captured backward
            with torch.no_grad():
                t = torch.empty_like(v).copy_(v)
            if v.requires_grad:
                t.requires_grad_(True)
            static_ins.append(t)
        torch.cuda.synchronize(self.device)
        self.params.prepare_backward()
        mod = self.stage_mods[stage]
        from ..ops import _lib
        n0 = _lib.launch_count()
        fwd = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fwd, pool=pool, capture_error_mode="thread_local"):
            with gen_amp_context(self.device, self.option.mixed_precision):
                outs = mod(*static_ins)
        if not isinstance(outs, (tuple, list)):
            outs = (outs,)
        outs = tuple(outs)
        grad_outs = [(j, torch.zeros_like(o)) for j, o in enumerate(outs)
                     if torch.is_tensor(o) and o.requires_grad]
        n1 = _lib.launch_count()
        bwd = None
        if grad_outs:
            for t in static_ins:
                if torch.is_tensor(t) and t.requires_grad and t.is_leaf and \
                        not self._is_param_view(t):
                    t.grad = None
            bwd = torch.cuda.CUDAGraph()
            with torch.cuda.graph(bwd, pool=pool,
                                  capture_error_mode="thread_local"):
                torch.autograd.backward([outs[j] for j, _ in grad_outs],
                                        [g for _, g in grad_outs])
        gs.fwd, gs.bwd = fwd, bwd
        gs.fwd_kernels, gs.bwd_kernels = n1 - n0, _lib.launch_count() - n1
        _lib.add_launches(-(gs.fwd_kernels + gs.bwd_kernels))   # recorded, not executed
        gs.static_ins, gs.static_outs, gs.grad_outs = static_ins, outs, grad_outs

    def _is_param_view(self, t: torch.Tensor) -> bool:
        ptrs = getattr(self, "_param_ptrs", None)
        if ptrs is None:
            ptrs = {s.view.data_ptr() for s in self.params.slots.values()
                    if torch.is_tensor(s.view)}
            self._param_ptrs = ptrs
        return t.data_ptr() in ptrs

    def send_act(self, comm: CommPlan, stage: int, mb: int) -> None:
        outs = self.fw_outputs[(stage, mb)]
        for m in comm.send_at.get((int(StepWork.SEND_ACT), stage, mb), []):
            self._send(m, outs[m.key[2]])
        sp = self.part.stages[stage]
        sink = [(j, outs[j]) for j, o in enumerate(sp.outputs)
                if any(c[0] == OUTSIDE for c in o.consumers)]
        if sink and self.runner is not None:
            self.runner.return_output(mb, stage, sink)

    def backward(self, comm: CommPlan, stage: int, mb: int) -> None:
        sp = self.part.stages[stage]
        outs = self.fw_outputs.pop((stage, mb))
        grads_by_out: Dict[int, torch.Tensor] = {}
        owned: set = set()      # outputs whose running sum lives in one of our receive buffers
        for m in comm.need_at.get((int(StepWork.RECV_GRAD), stage, mb), []):
            g = self._take(m)
            j = m.key[2]
            if j not in grads_by_out:
                grads_by_out[j] = g
                if m.src_rank != m.dst_rank:
                    owned.add(j)
            elif j in owned and grads_by_out[j].dtype == g.dtype:
                # an output with several consumers: sum in place in the first receive buffer
                # (it is ours until the next step's receive overwrites it)
                grads_by_out[j].add_(g)
            else:
                grads_by_out[j] = grads_by_out[j] + g
        if any(c[0] == OUTSIDE for o in sp.outputs for c in o.consumers):
            ev = self.bw_events.get(mb)
            if ev is not None:
                if not ev.wait(self.option.ctrl_timeout):
                    raise TimeoutError(f"exec_fn of micro-batch {mb} did not finish its backward")
                for j, g in self.loss_grads.get(mb, {}).items():
                    if g is not None:
                        g = g.to(self.device)
                        grads_by_out[j] = g if j not in grads_by_out else grads_by_out[j] + g
        tensors, grads = [], []
        for j, o in enumerate(outs):
            if not (torch.is_tensor(o) and o.requires_grad):
                continue
            g = grads_by_out.get(j)
            if g is None:
                continue   # nobody sent a gradient: contributes nothing
            if g.dtype != o.dtype:
                g = g.to(o.dtype)
            tensors.append(o)
            grads.append(g.reshape(o.shape))
        start = self.recorder.record_event(self.device)
        gs = self.graphs.get(self.graph_key.get((stage, mb))) if self.use_graphs else None
        if gs is not None and not gs.failed and gs.static_outs is outs:
            if gs.bwd is not None:
                for j, buf in gs.grad_outs:
                    g = grads_by_out.get(j)
                    if g is None:
                        buf.zero_()
                    else:
                        buf.copy_(g.reshape(buf.shape), non_blocking=True)
                self._wait_sends_from([getattr(t, "grad", None) for t in gs.static_ins
                                       if torch.is_tensor(t) and t.is_leaf])
                gs.bwd.replay()
                _lib_add(gs.bwd_kernels)
        elif tensors:
            self.params.prepare_backward()
            torch.autograd.backward(tensors, grads)
        self.recorder.append_bw(stage, start, self.recorder.record_event(self.device))

    def send_grad(self, comm: CommPlan, stage: int, mb: int) -> None:
        ins = self.fw_inputs.pop((stage, mb))
        for m in comm.send_at.get((int(StepWork.SEND_GRAD), stage, mb), []):
            t = ins[m.key[4]]
            g = t.grad if torch.is_tensor(t) else None
            if g is None:      # the stage did not use this input: its gradient is zero
                g = self.zero_bufs.get(m.key)
                if g is None:
                    g = torch.zeros(m.meta.size, dtype=m.meta.dtype, device=self.device)
                    self.zero_bufs[m.key] = g
            self._send(m, g)

    # ------------------------------------------------------------------ optimizer step
    def init_reducer(self, make_group: Callable[[Tuple[int, ...]], Any]) -> None:
        """One group per distinct set of pp ranks sharing a parameter."""
        sets = sorted({tuple(r) for r in self.part.shared_states.values()})
        for ranks in sets:
            g = make_group(ranks)
            if self.pp_rank in ranks:
                self.shared_groups[ranks] = g

    def all_reduce_shared_grads(self) -> None:
        for ph, ranks in sorted(self.part.shared_states.items()):
            if self.pp_rank not in ranks:
                continue
            slot = self.params.slots[ph]
            g = self.shared_groups.get(tuple(ranks))
            if g is None or slot.grad is None:
                continue
            g.all_reduce_sum(slot.grad)

    def optimizer_step(self) -> None:
        ev0 = self.recorder.record_event(self.device)
        self._optimizer_step()
        self.opt_events = (ev0, self.recorder.record_event(self.device))
        self.opt_event_log.append(self.opt_events)
        if len(self.opt_event_log) > 4096:      # nobody is reading them: keep the tail
            del self.opt_event_log[:2048]
            self.recorder.reset()

    def time_report(self, reset: bool = True) -> Dict[str, float]:
        """Device time this rank spent in stage forwards, stage backwards and optimizer steps
        since the last report (CUDA events on the compute stream; waits for incoming transfers
        are enqueued before a stage's first event and so are not counted), and the number of
        optimizer steps that covers.  The idle share of a step (pipeline bubble) follows from
        these and the step time."""
        fw, bw = self.recorder.get_event_logs()
        if self.device.type == "cuda" and self.opt_event_log:
            self.opt_event_log[-1][1].synchronize()
        rep = {"pp_rank": self.pp_rank,
               "fwd_ms": float(sum(sum(v) for v in fw.values())),
               "bwd_ms": float(sum(sum(v) for v in bw.values())),
               "opt_ms": float(sum(a.elapsed_time(b) for a, b in self.opt_event_log)),
               "steps": len(self.opt_event_log)}
        if reset:
            self.recorder.reset()
            self.opt_event_log.clear()
        return rep

    def last_optimizer_ms(self) -> float:
        """Device time of the last optimizer step (data-parallel reduce + update + gather); it
        runs after the last backward, so all of it is exposed."""
        ev = getattr(self, "opt_events", None)
        if ev is None:
            return 0.0
        if self.device.type == "cuda":
            ev[1].synchronize()
        return float(ev[0].elapsed_time(ev[1]))

    def _optimizer_step(self) -> None:
        self.all_reduce_shared_grads()
        grad_scale = 1.0
        fp16 = self.scaler.enabled
        if self.dp is not None and self.dp.fused:
            agreed = False
            if fp16 and self.inf_sync_job_wide:
                # a pipeline of several ranks: the skip decision must be the same on every rank
                # of the job, not only among the replicas of this stage.  A non-finite term
                # makes the reduced sum non-finite, so the local buckets decide.
                self.params.check_finite()
                self.sync_found_inf()
                agreed = True
            self.dp.reduce_and_step(self.params, self.scaler, fp16, found_agreed=agreed)
            self.gathered_stages.clear()    # 16-bit weight matrices are row-sharded again
            return
        if self.dp is not None:
            self.dp.all_reduce(self.params)
            grad_scale = 1.0 / self.dp.size
        if fp16:
            self.params.check_finite()
            self.sync_found_inf()
        self.params.step(grad_scale, self.scaler.scale_tensor, use_found_inf=fp16)
        if fp16:
            self.scaler.update(self.params.found_inf)

    def sync_found_inf(self) -> None:
        """Hook: OR the non-finite flag over every rank of the job (installed by the runtime
        front-end, which owns the process groups)."""
        return

    # ------------------------------------------------------------------ program driver
    def run(self, training: bool = True) -> None:
        steps = self.steps if training else self.eval_steps
        comm = self.comm if training else self.eval_comm
        if training and self.use_graphs and not self._captured_upfront and \
                self.train_steps_done >= self.graph_warmup_steps and \
                os.environ.get("PF_GRAPH_CAPTURE", "upfront") != "lazy":
            self.capture_all()
        if self.is_main:
            self.distribute_inputs(comm)
        ctx = contextlib.nullcontext() if training else torch.no_grad()
        nvtx = self.device.type == "cuda"
        with ctx:
            for st in steps:
                if nvtx:
                    torch.cuda.nvtx.range_push(f"DEV{self.pp_rank}_{st}")
                w, s, b = st.work, st.node_id, st.batch_id
                if w == StepWork.RECV_ACT:
                    self._receive(comm, comm.need_at.get((int(w), s, b), []))
                elif w == StepWork.FORWARD:
                    self.forward(comm, s, b)
                elif w == StepWork.SEND_ACT:
                    self.send_act(comm, s, b)
                elif w == StepWork.RECV_GRAD:
                    self._receive(comm, comm.need_at.get((int(w), s, b), []))
                elif w == StepWork.BACKWARD:
                    self.backward(comm, s, b)
                elif w == StepWork.SEND_GRAD:
                    self.send_grad(comm, s, b)
                elif w == StepWork.OPTIMIZER_STEP and training:
                    self.optimizer_step()
                    self.train_steps_done += 1
                    if nvtx and self.params is not None and self.params.native:
                        # a kernel that gave up on a bounded wait (a replica that is late or
                        # gone) ends the job here, one step later, without a host sync per step
                        from ..ops import kernels as kx
                        kx.poll_status(self.device)
                if nvtx:
                    torch.cuda.nvtx.range_pop()
        if not training:
            self.fw_inputs.clear()
            self.fw_outputs.clear()

    # ------------------------------------------------------------------ reporting
    def memory_usage(self) -> Dict[str, float]:
        if self.device.type != "cuda":
            return {"idle": 0.0, "max": 0.0, "alloc": 0.0, "reserved": 0.0}
        mx = torch.cuda.max_memory_allocated(self.device)
        return {"idle": self.idle_mem, "max": mx, "alloc": mx - self.idle_mem,
                "reserved": torch.cuda.memory_reserved(self.device)}

    def log_memory_usage(self) -> None:
        m = self.memory_usage()
        self.log.info("[Worker %d] memory usage: idle: %s, max: %s, alloc: %s, reserved: %s",
                      self.pp_rank, fmem(m["idle"]), fmem(m["max"]), fmem(m["alloc"]),
                      fmem(m["reserved"]))
