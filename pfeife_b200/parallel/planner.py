"""Planner: split points, schedule parameters and the PPxDP mesh from measured per-segment
latency / memory and the link model.

Behavioural counterpart of pfeife/schedule/planner.py:540-1997:
  * ``gen_graph(batch_cnt, max_mem, split_points)`` tries stage counts ``loop_cnt * D`` (or
    ``{1,2,3} * D`` when ``loop_cnt`` is not fixed) x every ``PipeSchedSet`` candidate; for each
    it seeds split points that balance time under the memory cap, then improves them with a
    width-2 beam search (<= ``BEAM_ITER`` rounds; moves: shift one point by up to +-10 segments,
    or rescale all points about one), scoring candidates by the simulated makespan and rejecting
    those whose predicted peak memory exceeds ``RESERVE_MEM_RATIO`` x device memory;
  * a deeper loop level is kept only when it improves the step time by >= 1 %, and looping is not
    tried when the mean stage forward is below ``FWD_AVG_MIN`` ms;
  * ``DependencyGraph`` is the DAG of compute and transfer nodes of the chosen plan with the
    per-channel transfer order the runtime replays.
Additions: a data-parallel cost term and ``choose_mesh`` which enumerates (PP, DP)
factorizations of the GPU count and picks the one with the best predicted samples/s.
The candidate evaluator has a C++ implementation (csrc/planner_eval.cpp) that is used when the
host library is built; the Python simulation in pipe_graph.py is the oracle.
"""
from __future__ import annotations

import itertools
import math
import random
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from ..graph.comp_graph import CompGraph
from ..utils import fmem, get_logger
from .device_bench import DeviceBench
from .pipe_graph import RESERVE_MEM_RATIO, PipeEdge, PipeGraph, PipeNode, Simulation
from .schedule import PipeSchedParams, PipeSchedSet

RAND_WALK_ITER = 1000
BEAM_ITER = 100
BEAM_WIDTH = 2
FWD_AVG_MIN = 3.0
T_MAX_EPSILON = 1e-6
IMPROVE_MIN = 0.01


# ------------------------------------------------------------------------------ dependency graph
@dataclass
class SchedNode:
    id: int
    rank: int
    duration: float = 0.0
    start: float = 0.0
    prev: List[int] = field(default_factory=list)
    next: List[int] = field(default_factory=list)


@dataclass
class SchedCompNode(SchedNode):
    stage: int = 0
    batch: int = 0
    is_fwd: bool = True


@dataclass
class SchedCommNode(SchedNode):
    src_stage: int = 0
    dst_stage: int = 0
    batch: int = 0
    is_grad: bool = False
    dst_rank: int = 0
    nonstd: bool = False      # skip connection (not stage i -> i+-1)


class DependencyGraph:
    """Compute and transfer nodes of a plan.  ``calc_schedule`` fills start times and returns
    ``(max_time, channel_comms)`` where ``channel_comms[(src_rank, dst_rank)]`` is the total
    order of transfers on that directed channel."""

    def __init__(self, pipe_graph: PipeGraph, sched: PipeSchedParams):
        self.pipe_graph = pipe_graph
        self.sched = sched
        self.comp: Dict[Tuple[int, int, bool], SchedCompNode] = {}
        self.comm: Dict[Tuple[bool, int, int, int], SchedCommNode] = {}
        self.nodes: List[SchedNode] = []
        self.max_time = 0.0
        self.channel_comms: Dict[Tuple[int, int], List[Tuple[bool, int, int, int]]] = {}
        self._build()

    def _new(self, node: SchedNode) -> SchedNode:
        node.id = len(self.nodes)
        self.nodes.append(node)
        return node

    def _link(self, a: SchedNode, b: SchedNode) -> None:
        a.next.append(b.id)
        b.prev.append(a.id)

    def _build(self) -> None:
        pg = self.pipe_graph
        for r, works in enumerate(self.sched.rank_works):
            prev = None
            for s, b, f in works:
                n = pg.nodes[s]
                node = self._new(SchedCompNode(0, r, n.comp_time if f else n.back_time,
                                               stage=s, batch=b, is_fwd=f))
                self.comp[(s, b, f)] = node
                if prev is not None:
                    self._link(prev, node)
                prev = node
        for e in pg.edges:
            self.add_comm(e)

    def add_comm(self, e: PipeEdge) -> None:
        """Transfer nodes of one stage-to-stage edge, every micro-batch, both directions."""
        pg = self.pipe_graph
        ra, rb = pg.nodes[e.start].rank, pg.nodes[e.end].rank
        nonstd = e.end != e.start + 1
        for b in range(self.sched.batch_cnt):
            for grad in (False, True):
                src, dst = (e.end, e.start) if grad else (e.start, e.end)
                r_src, r_dst = (rb, ra) if grad else (ra, rb)
                c = self._new(SchedCommNode(0, r_src, 0.0 if ra == rb else e.send_time,
                                            src_stage=src, dst_stage=dst, batch=b, is_grad=grad,
                                            dst_rank=r_dst, nonstd=nonstd))
                self.comm[(grad, src, dst, b)] = c
                self._link(self.comp[(src, b, not grad)], c)
                self._link(c, self.comp[(dst, b, not grad)])

    add_nonstd_comm = add_comm

    def calc_schedule(self) -> Tuple[float, Dict[Tuple[int, int], List[Tuple[bool, int, int, int]]]]:
        sim = self.pipe_graph.simulate(self.sched, record=True)
        for key, t in sim.start_times.items():
            self.comp[key].start = t
        self.max_time = sim.makespan
        self.channel_comms = sim.channel_order
        return self.max_time, self.channel_comms

    # compact, id-based form for shipping to workers
    def serialize(self) -> dict:
        return {"sched": self.sched.key(), "max_time": self.max_time,
                "channel_comms": {k: list(v) for k, v in self.channel_comms.items()}}


# ------------------------------------------------------------------------------ stage building
def _link_time(bench: Optional[DeviceBench], r1: int, r2: int, nbytes: float) -> float:
    if bench is None or r1 == r2:
        return 0.0
    return bench.send_time_rank(r1, r2, nbytes)


class _Prefix:
    """Prefix sums of the per-segment statistics for O(1) stage aggregation."""

    def __init__(self, cg: CompGraph):
        self.n = len(cg.nodes)
        z = [0.0]
        self.t = list(itertools.accumulate((n.comp_time for n in cg.nodes), initial=0.0))
        self.bt = list(itertools.accumulate(
            (n.back_time if n.back_time is not None else n.comp_time * cg.fb_ratio
             for n in cg.nodes), initial=0.0))
        self.w = list(itertools.accumulate((float(n.weight) for n in cg.nodes), initial=0.0))
        self.pb = list(itertools.accumulate((float(n.param_bytes) for n in cg.nodes), initial=0.0))
        self.a = list(itertools.accumulate((float(n.act_mem) for n in cg.nodes), initial=0.0))
        self.o = list(itertools.accumulate((float(n.optim_time) for n in cg.nodes), initial=0.0))
        self.temp = [float(n.temp_mem) for n in cg.nodes]
        self.act = [float(n.act_mem) for n in cg.nodes]


def build_pipe_graph(cg: CompGraph, split_points: Sequence[int], device_cnt: int,
                     bench: Optional[DeviceBench], batch_cnt: int,
                     prefix: Optional[_Prefix] = None) -> PipeGraph:
    """Stages, edges and static I/O buffer sizes for a set of split points
    (pfeife/schedule/planner.py:1271-1370)."""
    px = prefix or _Prefix(cg)
    bounds = cg.stage_bounds(split_points)
    nodes: List[PipeNode] = []
    for s, (lo, hi) in enumerate(bounds):
        # transient peak of the stage forward: activations accumulated so far + the worst
        # segment transient on top
        run = 0.0
        temp = 0.0
        for i in range(lo, hi):
            temp = max(temp, run + px.temp[i])
            run += px.act[i]
        nodes.append(PipeNode(s, s % device_cnt, lo, hi, weight=px.w[hi] - px.w[lo],
                              param_bytes=px.pb[hi] - px.pb[lo], act_mem=px.a[hi] - px.a[lo],
                              temp_mem=max(temp, px.a[hi] - px.a[lo]),
                              comp_time=px.t[hi] - px.t[lo], back_time=px.bt[hi] - px.bt[lo],
                              optim_time=px.o[hi] - px.o[lo]))
    edges: List[PipeEdge] = []
    io = [0.0] * device_cnt
    for (a, b), nbytes in sorted(cg.cross_edges(bounds).items()):
        ra, rb = a % device_cnt, b % device_cnt
        edges.append(PipeEdge(a, b, float(nbytes), _link_time(bench, ra, rb, nbytes)))
        if ra != rb:
            io[rb] += nbytes * batch_cnt * 3   # receive buffer + clone + its gradient
            io[ra] += nbytes * batch_cnt * 2   # gradient receive buffer + send staging
    return PipeGraph(nodes, edges, device_cnt, io)


@dataclass
class Plan:
    split_points: List[int]
    sched: PipeSchedParams
    pipe_graph: PipeGraph
    time: float
    peak_mem: List[float]
    dep_graph: Optional[DependencyGraph] = None
    sim: Optional[Simulation] = None


# ------------------------------------------------------------------------------ generators
class PipeGraphGenerator:
    """Base generator: manual split points, or a search implemented by ``_optimize_split``.
    This base class implements the simple strategies (``same_time``, ``same_mem``,
    ``random_walk``) that the reference lists but ships broken."""

    strategy = "same_time"

    def __init__(self, comp_graph: CompGraph, device_bench: Optional[DeviceBench], option):
        self.cg = comp_graph
        self.bench = device_bench
        self.option = option
        self.device_cnt = option.device_cnt
        self.px = _Prefix(comp_graph)
        self.log = get_logger()
        self.evals = 0

    # ---- evaluation of one candidate
    def _valuate_points(self, points: Sequence[int], sched: PipeSchedParams,
                        max_mem: Optional[Sequence[float]]) -> Tuple[float, bool, PipeGraph]:
        self.evals += 1
        pg = build_pipe_graph(self.cg, points, self.device_cnt, self.bench, sched.batch_cnt,
                              self.px)
        feasible = True if max_mem is None else pg.fits(sched, max_mem)
        return pg.get_value(sched), feasible, pg

    # ---- seeds
    def _balanced_points(self, node_cnt: int, by: str = "time") -> List[int]:
        n = self.px.n
        node_cnt = min(node_cnt, n)
        acc = self.px.t if by == "time" else [w + a for w, a in zip(self.px.w, self.px.a)]
        total = acc[-1]
        pts: List[int] = []
        j = 1
        for s in range(1, node_cnt):
            target = total * s / node_cnt
            while j < n - (node_cnt - s) and acc[j] < target:
                j += 1
            j = max(j, (pts[-1] + 1) if pts else 1)
            pts.append(min(j, n - (node_cnt - s)))
        return pts

    def _get_initial_split_points(self, node_cnt: int, sched: PipeSchedParams,
                                  max_mem: Optional[Sequence[float]]) -> List[int]:
        pts = self._balanced_points(node_cnt, "time")
        if max_mem is not None:
            _, ok, _ = self._valuate_points(pts, sched, max_mem)
            if not ok:
                alt = self._balanced_points(node_cnt, "mem")
                if self._valuate_points(alt, sched, max_mem)[1]:
                    return alt
        return pts

    def _optimize_split(self, points: List[int], sched: PipeSchedParams,
                        max_mem: Optional[Sequence[float]]) -> Tuple[float, List[int], bool]:
        if self.strategy == "same_mem":
            points = self._balanced_points(len(points) + 1, "mem")
        if self.strategy == "random_walk":
            return self._random_walk(points, sched, max_mem)
        v, ok, _ = self._valuate_points(points, sched, max_mem)
        return v, list(points), ok

    def _random_walk(self, points, sched, max_mem):
        rng = random.Random(self.option.bench_seed)
        best_v, best_ok, _ = self._valuate_points(points, sched, max_mem)
        best = list(points)
        for _ in range(RAND_WALK_ITER if points else 0):
            cand = list(best)
            i = rng.randrange(len(cand))
            cand[i] += rng.choice([-3, -2, -1, 1, 2, 3])
            if not _valid(cand, self.px.n):
                continue
            v, ok, _ = self._valuate_points(cand, sched, max_mem)
            if (ok and not best_ok) or (ok == best_ok and v < best_v):
                best, best_v, best_ok = cand, v, ok
        return best_v, best, best_ok

    # ---- main entry
    def _stage_counts(self) -> List[int]:
        D = self.device_cnt
        if self.option.loop_cnt:
            return [self.option.loop_cnt * D]
        return [D, 2 * D, 3 * D]

    def _candidates(self, batch_cnt: int, node_cnt: int) -> List[PipeSchedParams]:
        scheds = PipeSchedSet(self.device_cnt, batch_cnt, node_cnt).scheds
        o = self.option
        if o.loop_batch is not None:
            f = [s for s in scheds if s.loop_batch == o.loop_batch]
            scheds = f or [PipeSchedParams(self.device_cnt, batch_cnt, node_cnt,
                                           min(batch_cnt, max(o.loop_batch, 1)), 0)]
        if o.prefetch_fwd is not None:
            f = [s for s in scheds if s.prefetch_fwd == o.prefetch_fwd]
            scheds = f or [PipeSchedParams(self.device_cnt, batch_cnt, node_cnt,
                                           scheds[0].loop_batch, o.prefetch_fwd)]
        return scheds

    def gen_graph(self, batch_cnt: int, max_mem: Optional[Sequence[float]] = None,
                  split_points: Optional[Sequence[int]] = None) -> Plan:
        """-> the best plan found (``.pipe_graph``, ``.sched``, ``.dep_graph``)."""
        t_begin = time.perf_counter()
        D = self.device_cnt
        n_seg = self.px.n
        best: Optional[Plan] = None

        def consider(points, sched, v, ok, pg):
            nonlocal best
            better = best is None or (ok and not best._ok) or (ok == best._ok and v < best.time)
            if better:
                best = Plan(list(points), sched, pg, v, pg.get_peak_memory(sched))
                best._ok = ok

        if split_points is not None:
            split_points = sorted(int(p) for p in split_points)
            if not _valid(split_points, n_seg):
                raise ValueError(f"split points {split_points} invalid for {n_seg} segments")
            node_cnt = len(split_points) + 1
            for sched in self._candidates(batch_cnt, node_cnt):
                v, ok, pg = self._valuate_points(split_points, sched, max_mem)
                consider(split_points, sched, v, ok, pg)
        else:
            prev_level_best = math.inf
            for level, node_cnt in enumerate(self._stage_counts()):
                if node_cnt > n_seg:
                    break
                if level > 0 and not self.option.loop_cnt:
                    if self.px.t[-1] / node_cnt <= FWD_AVG_MIN:
                        self.log.info("mean stage forward %.3f ms <= %.1f ms: not looping further",
                                      self.px.t[-1] / node_cnt, FWD_AVG_MIN)
                        break
                level_best = math.inf
                for sched in self._candidates(batch_cnt, node_cnt):
                    init = self._get_initial_split_points(node_cnt, sched, max_mem)
                    self.log.debug("initial split points for %d nodes: %s", node_cnt, init)
                    v, pts, ok = self._optimize_split(init, sched, max_mem)
                    _, _, pg = self._valuate_points(pts, sched, max_mem)
                    self.log.debug("test %s -> %.4f %s %s", sched, v, pts, ok)
                    consider(pts, sched, v, ok, pg)
                    if ok:
                        level_best = min(level_best, v)
                if level > 0 and level_best > prev_level_best * (1.0 - IMPROVE_MIN):
                    break
                prev_level_best = min(prev_level_best, level_best)
        assert best is not None, "no schedule candidate"
        if not best._ok and max_mem is not None:
            self.log.warning("no memory-feasible plan found; using the fastest infeasible one")
        self._refine_dep_graph(best)
        self.log.info("elapsed time: %.2fs (%d evaluations), result: %s",
                      time.perf_counter() - t_begin, self.evals, best.time)
        self.log.info("split points: %s, expect time: %s, schedule: %s", best.split_points,
                      best.time, best.sched)
        idle = best.pipe_graph.idle_memory()
        for r, (i, p) in enumerate(zip(idle, best.peak_mem)):
            self.log.info("dev %d - idle mem: %s peak: %s", r, fmem(i), fmem(p))
        if self.option.print_graph:
            self.log.info("%s", best.pipe_graph.describe())
        return best

    def plan_from(self, split_points: Sequence[int], sched_key: Sequence[int],
                  max_mem: Optional[Sequence[float]] = None) -> Plan:
        """The plan for given split points and schedule parameters
        (``PipeSchedParams.key()``), without any search: what a data-parallel replica installs
        after the first replica has planned."""
        sched = PipeSchedParams(*[int(v) for v in sched_key])
        pts = [int(p) for p in split_points]
        v, ok, pg = self._valuate_points(pts, sched, max_mem)
        plan = Plan(pts, sched, pg, v, pg.get_peak_memory(sched))
        plan._ok = ok
        self._refine_dep_graph(plan)
        return plan

    def _refine_dep_graph(self, plan: Plan) -> None:
        dg = DependencyGraph(plan.pipe_graph, plan.sched)
        dg.calc_schedule()
        plan.dep_graph = dg
        plan.sim = plan.pipe_graph.simulate(plan.sched)


def _valid(points: Sequence[int], n_seg: int) -> bool:
    prev = 0
    for p in points:
        if p <= prev or p >= n_seg:
            return False
        prev = p
    return True


class BeamSingleGenerator(PipeGraphGenerator):
    """Width-2 beam search, one split point moved per step (the default, ``beam_single``)."""

    strategy = "beam_single"
    max_shift = 10

    def _neighbours(self, pts: List[int]) -> Iterable[List[int]]:
        n = self.px.n
        for i in range(len(pts)):
            for d in itertools.chain(range(1, self.max_shift + 1)):
                for sgn in (-1, 1):
                    c = list(pts)
                    c[i] += sgn * d
                    if _valid(c, n):
                        yield c
        # rescale every point about point i (keeps i, stretches/compresses the rest)
        for i in range(len(pts)):
            for f in (0.9, 1.1):
                c = [int(round(pts[i] + (p - pts[i]) * f)) for p in pts]
                if c != pts and _valid(c, n):
                    yield c

    def _optimize_split(self, points, sched, max_mem):
        if not points:
            v, ok, _ = self._valuate_points(points, sched, max_mem)
            return v, [], ok
        seen = {tuple(points)}
        v0, ok0, _ = self._valuate_points(points, sched, max_mem)
        beam: List[Tuple[bool, float, List[int]]] = [(not ok0, v0, list(points))]
        for it in range(BEAM_ITER):
            cand = list(beam)
            for _bad, _v, pts in beam:
                for c in self._neighbours(pts):
                    key = tuple(c)
                    if key in seen:
                        continue
                    seen.add(key)
                    v, ok, _ = self._valuate_points(c, sched, max_mem)
                    cand.append((not ok, v, c))
            cand.sort(key=lambda x: (x[0], x[1]))
            new_beam = cand[:BEAM_WIDTH]
            self.log.debug("beam %d - %s", it, " - ".join(f"{v} / {p} {not bad}"
                                                           for bad, v, p in new_beam))
            if [b[2] for b in new_beam] == [b[2] for b in beam]:
                break
            beam = new_beam
        bad, v, pts = beam[0]
        return v, pts, not bad


class BeamSearchGenerator(BeamSingleGenerator):
    """``beam_2``: wider shifts (+-15) and two points moved together."""

    strategy = "beam_2"
    max_shift = 15

    def _neighbours(self, pts):
        yield from super()._neighbours(pts)
        n = self.px.n
        for i in range(len(pts) - 1):
            for d in (-4, -2, 2, 4):
                c = list(pts)
                c[i] += d
                c[i + 1] += d
                if _valid(c, n):
                    yield c


class SameMemGenerator(PipeGraphGenerator):
    strategy = "same_mem"


class RandomWalkGenerator(PipeGraphGenerator):
    strategy = "random_walk"


_GENERATORS = {
    "beam_single": BeamSingleGenerator, "beam_2": BeamSearchGenerator,
    "random_walk": RandomWalkGenerator, "same_mem": SameMemGenerator,
    "same_time": PipeGraphGenerator,
}


def get_pipe_class(name: str):
    try:
        return _GENERATORS[name]
    except KeyError:
        raise ValueError(f"unknown partitioner {name!r}") from None


# ------------------------------------------------------------------------------ DP term + mesh
# Measured copy bandwidth of one B200's HBM3e (bytes/s); only used to estimate the optimizer
# step when the profile carries no measured optimizer time.
HBM_BYTES_PER_S = 6.5e12
# bytes the fused optimizer moves per parameter: gradient read + cleared, master, two moments
# read + written, 16-bit weight written
ADAM_BYTES_PER_PARAM = 34.0


def dp_exposed_time(param_bytes_per_rank: float, dp_size: int, bench: Optional[DeviceBench],
                    grad_dtype_bytes: int = 4, overlap: float = 0.0) -> float:
    """Predicted exposed time (ms) of the data-parallel step of one rank beyond its local
    optimizer: every rank reads the other ranks' gradients of its shard (``(dp-1)/dp`` of the
    gradient bytes cross the links towards it) and pushes its updated 16-bit weights to the
    others (the same share of 2 bytes per parameter leaves it; fp32 masters stay with their
    owner); reads and pushes follow each other inside one kernel, so their times add.  The
    link model is the measured one when `bench` carries it.  ``overlap`` is the fraction
    hidden behind the backward."""
    if dp_size <= 1:
        return 0.0
    n_el = param_bytes_per_rank / 4.0
    share = (dp_size - 1) / dp_size
    moved = n_el * (grad_dtype_bytes + 2) * share
    if bench is None or not bench.params:
        ms = moved / (770e9) * 1e3 + 0.05
    else:
        ms = bench.send_time(next(iter(bench.params)), moved)
    return ms * (1.0 - overlap)


def optimizer_time(param_bytes_per_rank: float, dp_size: int, measured_ms: float = 0.0) -> float:
    """Time (ms) of the optimizer update of one rank: the measured value when the profile has
    one, else the bytes the fused update moves at HBM bandwidth.  Under data parallelism every
    rank updates only its shard."""
    if measured_ms > 0.0:
        return measured_ms / max(1, dp_size)
    n_el = param_bytes_per_rank / 4.0
    return n_el * ADAM_BYTES_PER_PARAM / max(1, dp_size) / HBM_BYTES_PER_S * 1e3


@dataclass
class MeshChoice:
    pp: int
    dp: int
    plan: Plan
    step_ms: float
    samples_per_s: float
    table: List[Tuple[int, int, float, float, bool]] = field(default_factory=list)

    @property
    def dp_mesh(self) -> str:
        return f"-{self.dp},{self.pp}" if self.dp > 1 else f"{self.pp}"


def choose_mesh(comp_graph: CompGraph, world_size: int, option, bench: Optional[DeviceBench],
                device_mem: float, batch_size: Optional[int] = None) -> MeshChoice:
    """Evaluates every (PP, DP) with PP * DP = world_size and returns the best by predicted
    samples/s = ``batch_size * batch_cnt * DP / (pipeline step + exposed DP time)``.
    ``batch_cnt`` is per pipeline, as everywhere in this framework."""
    import copy
    log = get_logger()
    bs = batch_size or option.batch_size
    best: Optional[MeshChoice] = None
    table = []
    for pp in range(1, world_size + 1):
        if world_size % pp:
            continue
        dp = world_size // pp
        opt = copy.copy(option)
        opt.device_cnt = pp
        if pp == 1:
            opt.loop_cnt = 1
        if pp > len(comp_graph.nodes):
            continue
        gen = get_pipe_class(option.partitioner)(comp_graph, bench, opt)
        old = gen.log.level
        gen.log.setLevel(max(old, 30))
        try:
            plan = gen.gen_graph(option.batch_cnt, [device_mem] * pp, None)
        finally:
            gen.log.setLevel(old)
        per_rank = max(sum(n.param_bytes for n in plan.pipe_graph.nodes if n.rank == r)
                       for r in range(pp))
        # ZeRO-style sharding divides the static optimizer footprint by dp
        ok = max(plan.peak_mem) < RESERVE_MEM_RATIO * device_mem
        # the pipeline makespan contains the optimizer only when the profile measured it; the
        # data-parallel shard of it is what remains exposed either way
        measured_opt = max(sum(n.optim_time for n in plan.pipe_graph.nodes if n.rank == r)
                           for r in range(pp))
        step = plan.time - measured_opt + optimizer_time(per_rank, dp, measured_opt) + \
            dp_exposed_time(per_rank, dp, bench)
        sps = bs * option.batch_cnt * dp / step * 1e3
        table.append((pp, dp, step, sps, ok))
        cand = MeshChoice(pp, dp, plan, step, sps)
        if best is None or (ok and not best._ok) or (ok == best._ok and sps > best.samples_per_s):
            best = cand
            best._ok = ok
    assert best is not None
    best.table = table
    for pp, dp, step, sps, ok in table:
        log.info("mesh PP=%d x DP=%d: step %.2f ms, %.1f samples/s%s", pp, dp, step, sps,
                 "" if ok else " (over memory)")
    log.info("chosen mesh: PP=%d x DP=%d (--dp_mesh \"%s\")", best.pp, best.dp, best.dp_mesh)
    return best
