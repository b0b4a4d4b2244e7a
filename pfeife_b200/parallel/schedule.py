"""Pipeline schedules: the parametrised 1F1B family, candidate enumeration and the expansion
into per-rank step programs.

Behavioural spec: pfeife/schedule/scheduler.py:34-151 (schedule family: stage ``i`` lives on
rank ``i % device_cnt``; micro-batches advance in windows of ``loop_batch``; a rank switches to
one-forward-one-backward after a warm-up whose length grows with its distance to the last stage
and with ``prefetch_fwd``) and :154-421 (step expansion).  The DFS variant here is a real 1F1B
(the reference indexes its per-rank lists by stage id and breaks for looped placements), and
evaluation (forward-only) programs exist for every scheduler.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

Work = Tuple[int, int, bool]  # (stage, micro-batch, is_forward)


class StepWork(IntEnum):
    SEND_ACT = 1
    RECV_ACT = 2
    FORWARD = 3
    SEND_GRAD = 4
    RECV_GRAD = 5
    BACKWARD = 6
    OPTIMIZER_STEP = 7


@dataclass(frozen=True)
class Step:
    work: StepWork
    node_id: int
    batch_id: int

    def __str__(self) -> str:
        return f"{self.work.name}:{self.node_id}:{self.batch_id}"


class PipeSchedParams:
    """One member of the schedule family; ``rank_works[r]`` is rank r's ordered work list."""

    def __init__(self, device_cnt: int, batch_cnt: int, node_cnt: int, loop_batch: int,
                 prefetch_fwd: int):
        if batch_cnt < loop_batch:
            raise ValueError("batch_cnt must be >= loop_batch")
        if device_cnt < 1 or node_cnt < 1 or loop_batch < 1:
            raise ValueError("device_cnt, node_cnt and loop_batch must be positive")
        self.device_cnt = device_cnt
        self.batch_cnt = batch_cnt
        self.node_cnt = node_cnt
        self.loop_batch = loop_batch
        self.prefetch_fwd = prefetch_fwd
        self.rank_works: List[List[Work]] = self._build()

    def rank_of(self, stage: int) -> int:
        return stage % self.device_cnt

    def stages_of(self, rank: int) -> List[int]:
        return list(range(rank, self.node_cnt, self.device_cnt))

    def _build(self) -> List[List[Work]]:
        D, B, N, LB = self.device_cnt, self.batch_cnt, self.node_cnt, self.loop_batch
        fwd: List[List[Tuple[int, int]]] = [[] for _ in range(D)]
        bwd: List[List[Tuple[int, int]]] = [[] for _ in range(D)]
        for lo in range(0, B, LB):
            window = range(lo, min(lo + LB, B))
            for s in range(N):
                fwd[s % D].extend((s, b) for b in window)
            for s in reversed(range(N)):
                bwd[s % D].extend((s, b) for b in window)
        works: List[List[Work]] = []
        for r in range(D):
            if not fwd[r]:
                works.append([])
                continue
            last_stage = max(s for s, _ in fwd[r])
            tail = N - last_stage                      # stages from this rank's last to the end
            earlier_loops = last_stage // D            # stages this rank runs before its last
            warmup = earlier_loops * LB + tail + min(tail - 1, self.prefetch_fwd)
            out: List[Work] = []
            nb = 0
            for i, (s, b) in enumerate(fwd[r]):
                out.append((s, b, True))
                if i + 1 >= warmup:
                    s2, b2 = bwd[r][nb]
                    out.append((s2, b2, False))
                    nb += 1
            out.extend((s2, b2, False) for s2, b2 in bwd[r][nb:])
            works.append(out)
        return works

    def key(self) -> Tuple[int, int, int, int, int]:
        return (self.device_cnt, self.batch_cnt, self.node_cnt, self.loop_batch, self.prefetch_fwd)

    def __str__(self) -> str:
        return (f"PipeSched(node_cnt={self.node_cnt}, loop_batch={self.loop_batch}, "
                f"prefetch_fwd={self.prefetch_fwd})")

    __repr__ = __str__


class PipeSchedSet:
    """Candidate ``(loop_batch, prefetch_fwd)`` pairs for a stage count
    (pfeife/schedule/scheduler.py:132-151): looped placements try every ``loop_batch`` in
    ``[device_cnt, batch_cnt]`` that equals ``device_cnt`` or divides ``batch_cnt``; non-looped
    ones use ``loop_batch = batch_cnt``; ``prefetch_fwd`` ranges over ``[0, device_cnt)``."""

    def __init__(self, device_cnt: int, batch_cnt: int, node_cnt: int):
        self.device_cnt, self.batch_cnt, self.node_cnt = device_cnt, batch_cnt, node_cnt
        self.scheds: List[PipeSchedParams] = []
        if node_cnt > device_cnt:
            lbs = [lb for lb in range(device_cnt, batch_cnt + 1)
                   if lb == device_cnt or batch_cnt % lb == 0]
        else:
            lbs = [batch_cnt]
        for lb in lbs:
            for pf in range(device_cnt):
                self.scheds.append(PipeSchedParams(device_cnt, batch_cnt, node_cnt, lb, pf))

    def builder(self, loop_batch: int, prefetch_fwd: int) -> PipeSchedParams:
        return PipeSchedParams(self.device_cnt, self.batch_cnt, self.node_cnt, loop_batch,
                               prefetch_fwd)


# ------------------------------------------------------------------------------ step programs
def _fwd_steps(stage: int, mb: int) -> List[Step]:
    return [Step(StepWork.RECV_ACT, stage, mb), Step(StepWork.FORWARD, stage, mb),
            Step(StepWork.SEND_ACT, stage, mb)]


def _bwd_steps(stage: int, mb: int) -> List[Step]:
    return [Step(StepWork.RECV_GRAD, stage, mb), Step(StepWork.BACKWARD, stage, mb),
            Step(StepWork.SEND_GRAD, stage, mb)]


def expand_works(works: Iterable[Work], forward_only: bool = False) -> List[Step]:
    steps: List[Step] = []
    for stage, mb, is_fwd in works:
        if is_fwd:
            steps.extend(_fwd_steps(stage, mb))
        elif not forward_only:
            steps.extend(_bwd_steps(stage, mb))
    return steps


class Scheduler:
    """Synchronous scheduler base: ``steps[rank]`` is the training program of a rank, ending in
    ``OPTIMIZER_STEP`` when the rank has any work."""

    def __init__(self, sched_params: PipeSchedParams, dep_graph=None):
        self.sched_params = sched_params
        self.dep_graph = dep_graph
        self.node_cnt = sched_params.node_cnt
        self.device_cnt = sched_params.device_cnt
        self.batch_cnt = sched_params.batch_cnt
        self.works: List[List[Work]] = self._build_works()
        self.steps: List[List[Step]] = self._build_steps()

    # subclasses either reorder works or override _build_steps
    def _build_works(self) -> List[List[Work]]:
        return [list(w) for w in self.sched_params.rank_works]

    def _build_steps(self) -> List[List[Step]]:
        out = []
        for w in self.works:
            s = expand_works(w)
            if s:
                s.append(Step(StepWork.OPTIMIZER_STEP, -1, -1))
            out.append(s)
        return out

    def get_train_steps(self, worker_id: int) -> List[Step]:
        return self.steps[worker_id] if worker_id < len(self.steps) else []

    def get_eval_steps(self, worker_id: int) -> List[Step]:
        if worker_id >= len(self.works):
            return []
        return expand_works(self.works[worker_id], forward_only=True)


class BeamScheduler(Scheduler):
    """Plain expansion of the schedule family member."""


class SingleCommScheduler(Scheduler):
    """Same programs as :class:`BeamScheduler`; carries the dependency graph whose per-pair
    transfer order the planner computed (the default scheduler)."""

    def __init__(self, sched_params: PipeSchedParams, dep_graph=None):
        super().__init__(sched_params, dep_graph)


class NoSkewScheduler(Scheduler):
    pass


class ForwardOnlyScheduler(Scheduler):
    def _build_steps(self) -> List[List[Step]]:
        out = []
        for w in self.works:
            s = expand_works(w, forward_only=True)
            if s:
                s.append(Step(StepWork.OPTIMIZER_STEP, -1, -1))
            out.append(s)
        return out


class BFSScheduler(Scheduler):
    """GPipe order: every forward of every micro-batch, then every backward."""

    def _build_works(self) -> List[List[Work]]:
        D, B, N = self.device_cnt, self.batch_cnt, self.node_cnt
        works: List[List[Work]] = [[] for _ in range(D)]
        for s in range(N):
            works[s % D].extend((s, b, True) for b in range(B))
        for s in reversed(range(N)):
            works[s % D].extend((s, b, False) for b in range(B))
        return works


class DFSScheduler(Scheduler):
    """Synchronous 1F1B: micro-batches in windows of ``device_cnt``, a rank starts alternating
    once ``tail`` forwards (its distance to the last stage) are in flight."""

    def _build_works(self) -> List[List[Work]]:
        D, B, N = self.device_cnt, self.batch_cnt, self.node_cnt
        return PipeSchedParams(D, B, N, min(B, D) if N > D else B, 0).rank_works


class PipelessScheduler(Scheduler):
    """No overlap at all: a stage runs all its micro-batches, then sends them."""

    def _build_steps(self) -> List[List[Step]]:
        D, B, N = self.device_cnt, self.batch_cnt, self.node_cnt
        out: List[List[Step]] = [[] for _ in range(D)]
        for s in range(N):
            prog = out[s % D]
            for b in range(B):
                prog += [Step(StepWork.RECV_ACT, s, b), Step(StepWork.FORWARD, s, b)]
            prog += [Step(StepWork.SEND_ACT, s, b) for b in range(B)]
        for s in reversed(range(N)):
            prog = out[s % D]
            for b in range(B):
                prog += [Step(StepWork.RECV_GRAD, s, b), Step(StepWork.BACKWARD, s, b)]
            prog += [Step(StepWork.SEND_GRAD, s, b) for b in range(B)]
        for prog in out:
            if prog:
                prog.append(Step(StepWork.OPTIMIZER_STEP, -1, -1))
        return out

    def _build_works(self) -> List[List[Work]]:
        return BFSScheduler._build_works(self)


_SCHEDULERS = {
    "single_comm": SingleCommScheduler, "beam": BeamScheduler, "bfs": BFSScheduler,
    "dfs": DFSScheduler, "pipeless": PipelessScheduler, "noskew": NoSkewScheduler,
    "forward_only": ForwardOnlyScheduler,
}


def get_scheduler_class(name: str):
    try:
        return _SCHEDULERS[name]
    except KeyError:
        raise ValueError(f"unknown scheduler {name!r}; choose from {sorted(_SCHEDULERS)}") from None


def validate_works(params: PipeSchedParams, works: Optional[Sequence[Sequence[Work]]] = None
                   ) -> None:
    """Invariants every schedule must satisfy: each (stage, mb) runs forward exactly once and
    backward exactly once on the owning rank, forward before backward."""
    works = params.rank_works if works is None else works
    seen: Dict[Tuple[int, int, bool], int] = {}
    for r, ws in enumerate(works):
        for i, (s, b, f) in enumerate(ws):
            assert s % params.device_cnt == r, f"stage {s} scheduled on rank {r}"
            assert (s, b, f) not in seen, f"duplicate {(s, b, f)}"
            seen[(s, b, f)] = i
            if not f:
                assert (s, b, True) in seen, f"backward before forward for {(s, b)}"
    assert len(seen) == 2 * params.node_cnt * params.batch_cnt
