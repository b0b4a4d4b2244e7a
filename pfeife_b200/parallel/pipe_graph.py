"""Stage-level graph and cost model.

``PipeNode`` = one pipeline stage (a contiguous slice of profiled segments), ``PipeEdge`` = the
tensors flowing between two stages (adjacent or skip), ``PipeGraph`` = stages + edges + the two
evaluators the planner needs (pfeife/graph/pipe_graph.py:10-314):

* ``get_peak_memory(sched)`` walks every rank's work list adding ``act_mem`` on a forward and
  releasing it on the backward, on top of the static weights and I/O buffers;
* ``get_value(sched)`` is the makespan of the schedule: an event simulation in which each rank
  executes its work list in order, a work item starts when its inputs have arrived, and every
  DIRECTED rank pair is a serial FIFO channel whose transfers take ``link(bytes)``.  (The
  reference treats each unordered pair as one channel; with one communicator per direction the
  two directions do not queue behind each other here.)  The FIFO order per channel is a
  by-product (``Simulation.channel_order``) and is what the runtime replays.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .schedule import PipeSchedParams

RESERVE_MEM_RATIO = 0.85


@dataclass
class PipeNode:
    idx: int
    rank: int
    lo: int
    hi: int
    weight: float = 0.0        # static bytes: parameters x4 (+ buffers)
    param_bytes: float = 0.0
    act_mem: float = 0.0
    temp_mem: float = 0.0
    comp_time: float = 0.0
    back_time: float = 0.0
    optim_time: float = 0.0

    @property
    def node_len(self) -> int:
        return self.hi - self.lo


@dataclass
class PipeEdge:
    start: int
    end: int
    weight: float              # bytes per micro-batch
    send_time: float = 0.0     # ms, 0 when both stages share a rank


@dataclass
class Simulation:
    makespan: float
    rank_busy: List[float]                     # compute ms per rank
    rank_end: List[float]
    # directed channel (src_rank, dst_rank) -> [(is_grad, src_stage, dst_stage, micro_batch)]
    channel_order: Dict[Tuple[int, int], List[Tuple[bool, int, int, int]]]
    start_times: Dict[Tuple[int, int, bool], float] = field(default_factory=dict)

    @property
    def bubble_fraction(self) -> float:
        """Idle share of the rank-time rectangle (the classic pipeline bubble)."""
        total = self.makespan * len(self.rank_busy)
        return 1.0 - sum(self.rank_busy) / total if total > 0 else 0.0


class PipeGraph:
    def __init__(self, nodes: List[PipeNode], edges: List[PipeEdge], device_cnt: int,
                 io_bytes: Optional[List[float]] = None):
        self.nodes = nodes
        self.edges = edges
        self.device_cnt = device_cnt
        self.io_bytes = io_bytes or [0.0] * device_cnt   # static comm buffers per rank
        self.producers: List[List[PipeEdge]] = [[] for _ in nodes]
        self.consumers: List[List[PipeEdge]] = [[] for _ in nodes]
        for e in edges:
            self.producers[e.end].append(e)
            self.consumers[e.start].append(e)

    # ------------------------------------------------------------------ memory
    def idle_memory(self) -> List[float]:
        mem = list(self.io_bytes)
        for n in self.nodes:
            mem[n.rank] += n.weight
        return mem

    def get_peak_memory(self, sched: PipeSchedParams) -> List[float]:
        idle = self.idle_memory()
        peaks = []
        for r, works in enumerate(sched.rank_works):
            cur = peak = idle[r] if r < len(idle) else 0.0
            for s, _b, fwd in works:
                n = self.nodes[s]
                if fwd:
                    peak = max(peak, cur + n.temp_mem)
                    cur += n.act_mem
                else:
                    peak = max(peak, cur + max(0.0, n.temp_mem - n.act_mem))
                    cur -= n.act_mem
            peaks.append(peak)
        return peaks

    def fits(self, sched: PipeSchedParams, max_mem: Sequence[float]) -> bool:
        return all(p < RESERVE_MEM_RATIO * m for p, m in zip(self.get_peak_memory(sched), max_mem))

    # ------------------------------------------------------------------ time
    def simulate(self, sched: PipeSchedParams, record: bool = False) -> Simulation:
        D = self.device_cnt
        works = sched.rank_works
        ptr = [0] * D
        now = [0.0] * D
        busy = [0.0] * D
        f_done: Dict[Tuple[int, int], float] = {}
        b_done: Dict[Tuple[int, int], float] = {}
        arrive: Dict[Tuple[bool, int, int, int], float] = {}
        chan_free: Dict[Tuple[int, int], float] = {}
        order: Dict[Tuple[int, int], List[Tuple[bool, int, int, int]]] = {}
        starts: Dict[Tuple[int, int, bool], float] = {}
        remaining = sum(len(w) for w in works)
        while remaining:
            progressed = False
            for r in range(D):
                while ptr[r] < len(works[r]):
                    s, b, fwd = works[r][ptr[r]]
                    t0 = now[r]
                    ok = True
                    if fwd:
                        for e in self.producers[s]:
                            a = arrive.get((False, e.start, s, b))
                            if a is None:
                                ok = False
                                break
                            t0 = max(t0, a)
                    else:
                        if (s, b) not in f_done:
                            ok = False
                        for e in self.consumers[s]:
                            a = arrive.get((True, e.end, s, b))
                            if a is None:
                                ok = False
                                break
                            t0 = max(t0, a)
                    if not ok:
                        break
                    n = self.nodes[s]
                    dur = n.comp_time if fwd else n.back_time
                    t1 = t0 + dur
                    busy[r] += dur
                    now[r] = t1
                    if record:
                        starts[(s, b, fwd)] = t0
                    if fwd:
                        f_done[(s, b)] = t1
                        outs = [(e, e.end) for e in self.consumers[s]]
                    else:
                        b_done[(s, b)] = t1
                        outs = [(e, e.start) for e in self.producers[s]]
                    for e, other in outs:
                        r2 = self.nodes[other].rank
                        key = (not fwd, s, other, b)
                        if r2 == r:
                            arrive[key] = t1
                        else:
                            ch = (r, r2)
                            t = max(t1, chan_free.get(ch, 0.0)) + e.send_time
                            chan_free[ch] = t
                            arrive[key] = t
                            order.setdefault(ch, []).append(key)
                    ptr[r] += 1
                    remaining -= 1
                    progressed = True
            if not progressed:
                raise RuntimeError("schedule deadlocks: a work item waits on an input that is "
                                   "never produced")
        ends = [now[r] + sum(n.optim_time for n in self.nodes if n.rank == r) for r in range(D)]
        return Simulation(max(ends) if ends else 0.0, busy, ends, order, starts)

    def get_value(self, sched: PipeSchedParams) -> float:
        """Makespan in ms.  Uses the C++ evaluator when the host library is built, otherwise
        the Python simulation above (the oracle)."""
        v = self._native_value(sched)
        return self.simulate(sched).makespan if v is None else v

    def _native_value(self, sched: PipeSchedParams) -> Optional[float]:
        import ctypes
        from ..ops import _lib
        host = _lib.host_lib()
        if host is None:
            return None
        fn = host.pf_sim_schedule
        fn.restype = ctypes.c_double
        cache = getattr(sched, "_flat", None)
        if cache is None:
            off, st, mb, fw = [0], [], [], []
            for works in sched.rank_works:
                for s, b, f in works:
                    st.append(s)
                    mb.append(b)
                    fw.append(1 if f else 0)
                off.append(len(st))
            cache = ((ctypes.c_int * len(off))(*off), (ctypes.c_int * len(st))(*st),
                     (ctypes.c_int * len(mb))(*mb), (ctypes.c_uint8 * len(fw))(*fw))
            sched._flat = cache
        n, D, E = len(self.nodes), self.device_cnt, len(self.edges)
        dbl = lambda xs: (ctypes.c_double * max(1, len(xs)))(*xs)
        ints = lambda xs: (ctypes.c_int * max(1, len(xs)))(*xs)
        optim = [0.0] * D
        for nd in self.nodes:
            optim[nd.rank] += nd.optim_time
        v = fn(D, n, sched.batch_cnt, dbl([x.comp_time for x in self.nodes]),
               dbl([x.back_time for x in self.nodes]), dbl(optim),
               ints([x.rank for x in self.nodes]), E, ints([e.start for e in self.edges]),
               ints([e.end for e in self.edges]),
               dbl([0.0 if self.nodes[e.start].rank == self.nodes[e.end].rank else e.send_time
                    for e in self.edges]),
               cache[0], cache[1], cache[2], cache[3], None)
        if v < 0:
            raise RuntimeError("schedule deadlocks: a work item waits on an input that is "
                               "never produced")
        return float(v)

    # ------------------------------------------------------------------ printing
    def describe(self) -> str:
        from ..utils import fmem
        lines = [f"GRAPH: {len(self.nodes)} nodes / {len(self.edges)} edges", "==== nodes ===="]
        for n in self.nodes:
            out_w = sum(e.weight for e in self.consumers[n.idx])
            lines.append(
                f"Node [{n.idx}/{n.rank}] (weight: {fmem(n.weight)}, act_mem: {fmem(n.act_mem)}, "
                f"temp_mem: {fmem(n.temp_mem)}, comp_time: {n.comp_time}, back_time: "
                f"{n.back_time}, optim_time: {n.optim_time}, node len: {n.node_len}, "
                f"send weight: {fmem(out_w)})")
        lines.append("==== edges ====")
        for e in self.edges:
            lines.append(f"Edge ({e.start} -> {e.end}) (weight: {fmem(e.weight)}, device: "
                         f"{self.nodes[e.start].rank} -> {self.nodes[e.end].rank}, send time: "
                         f"{e.send_time})")
        return "\n".join(lines)
