"""Computation graph: the captured FX graph linearised into profiled segments.

A ``CompGraph`` is a linear list of ``CompNode``s (each a run of consecutive FX nodes), the
tensor values flowing between them (``CompEdge``: bytes and shapes) and the parameter
placement (``ParamSet``).  Split points index this list.  It plays the role of
pfeife/graph/computation_graph.py:26-484; the per-segment statistics have the same meaning:
``weight`` = 4 x parameter bytes (weights, gradients, two Adam moments), ``act_mem`` = bytes a
forward leaves alive for the backward, ``temp_mem`` = transient peak during the forward,
``comp_time`` / ``optim_time`` in milliseconds, ``fb_ratio`` = backward / forward time.

Profile cache (``--graph_bench``): a pickle of ``{"format": "pfeife_b200.graph_bench/1",
"nodes": [...], "edges": [...], "fb_ratio": f}`` whose entries are copied positionally onto a
freshly captured graph, so a file is valid only for the same model, micro-batch size, dtype and
segmentation.  Files written by the reference (a pickled dummy ``CompGraph`` of its own classes,
pfeife/graph/computation_graph.py:379-484) are read through the same positional rule.
"""
from __future__ import annotations

import operator
import pickle
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

import torch
import torch.fx as fx

from .capture import CapturedGraph

# share of device memory above which the profiling pass moves what it keeps alive to the host
GRAPH_FETCH_MEM_CAP = 0.6
WEIGHT_MULTIPLIER = 4  # weights + gradients + two optimizer moments
FORMAT = "pfeife_b200.graph_bench/1"

_SHAPE_METHODS = {
    "view", "reshape", "transpose", "permute", "size", "unsqueeze", "squeeze", "flatten",
    "expand", "t", "dim", "unflatten", "chunk", "split", "unbind", "__getitem__", "stride",
    "numel", "view_as", "expand_as", "contiguous", "detach",
}
_SHAPE_FUNCTIONS = {operator.getitem, getattr, torch.transpose, torch.reshape, torch.permute,
                    torch.flatten, torch.unsqueeze, torch.squeeze}


@dataclass
class ShapeMeta:
    size: Tuple[int, ...]
    dtype: torch.dtype
    nbytes: int
    requires_grad: bool = True

    @staticmethod
    def of(t: torch.Tensor) -> "ShapeMeta":
        size = tuple(int(s) for s in t.shape)
        n = 1
        for s in size:
            n *= s
        return ShapeMeta(size, t.dtype, n * t.element_size(),
                         bool(t.requires_grad or t.dtype.is_floating_point))


def _tensor_leaves(v: Any) -> List[torch.Tensor]:
    if torch.is_tensor(v):
        return [v]
    if isinstance(v, (tuple, list)):
        out: List[torch.Tensor] = []
        for e in v:
            out.extend(_tensor_leaves(e))
        return out
    return []


def value_bytes(node: fx.Node) -> int:
    ex = node.meta.get("example_value", node.meta.get("val"))
    return sum(ShapeMeta.of(t).nbytes for t in _tensor_leaves(ex))


def is_trivial(node: fx.Node) -> bool:
    """Nodes that allocate nothing worth a segment of their own."""
    if node.op == "call_method" and node.target in _SHAPE_METHODS:
        return True
    if node.op == "call_function" and node.target in _SHAPE_FUNCTIONS:
        return True
    ex = node.meta.get("example_value", node.meta.get("val"))
    return ex is not None and not _tensor_leaves(ex)


@dataclass
class CompNode:
    idx: int
    fx_nodes: List[str]
    param_inputs: List[int] = field(default_factory=list)  # placeholder indices first used here
    param_bytes: int = 0
    weight: int = 0
    act_mem: int = 0
    temp_mem: int = 0
    comp_time: float = 1.0
    back_time: Optional[float] = None
    optim_time: float = 0.0
    out_bytes: int = 0

    @property
    def bwd_time(self) -> float:
        return self.back_time if self.back_time is not None else self.comp_time


@dataclass
class CompEdge:
    start: int               # producer segment
    end: int                 # consumer segment
    value: str               # FX node name of the value
    weight: int              # bytes
    shape: List[ShapeMeta] = field(default_factory=list)


@dataclass
class ParamSet:
    """Which segment first touches each state placeholder, and which placeholders are used by
    more than one segment (candidates for cross-stage sharing)."""
    first_use: Dict[int, int] = field(default_factory=dict)
    users: Dict[int, List[int]] = field(default_factory=dict)

    def shared_between(self, bounds: Sequence[Tuple[int, int]]) -> Dict[int, List[int]]:
        """placeholder index -> sorted stage ids using it, for placeholders used by >1 stage.
        ``bounds[s] = (lo, hi)`` is stage s's half-open segment range."""
        out: Dict[int, List[int]] = {}
        for ph, segs in self.users.items():
            stages = sorted({s for s, (lo, hi) in enumerate(bounds) for g in segs if lo <= g < hi})
            if len(stages) > 1:
                out[ph] = stages
        return out


class CompGraph:
    def __init__(self, captured: CapturedGraph):
        self.captured = captured
        self.nodes: List[CompNode] = []
        self.edges: List[CompEdge] = []
        self.param_set = ParamSet()
        self.fb_ratio: float = 2.0
        self.seg_of: Dict[str, int] = {}          # FX node name -> segment index
        self.input_users: Dict[int, List[int]] = {}   # user-input placeholder -> segments
        self.output_segments: List[int] = []      # segments producing model outputs
        self.placeholder_order: List[int] = []
        self._build()

    # ------------------------------------------------------------------ construction
    def _build(self) -> None:
        gm = self.captured.gm
        ph_index = {i.node_name: i for i in self.captured.inputs}
        compute = [n for n in gm.graph.nodes if n.op in ("call_function", "call_method",
                                                         "call_module", "get_attr")]
        # 1. segmentation: a non-trivial node opens a segment, trivial ones ride along
        cur: Optional[CompNode] = None
        pending: List[str] = []
        for n in compute:
            if is_trivial(n) or n.op == "get_attr":
                if cur is None:
                    pending.append(n.name)
                else:
                    cur.fx_nodes.append(n.name)
                    self.seg_of[n.name] = cur.idx
                continue
            cur = CompNode(len(self.nodes), pending + [n.name])
            pending = []
            for name in cur.fx_nodes:
                self.seg_of[name] = cur.idx
            self.nodes.append(cur)
        if pending:
            if cur is None:
                cur = CompNode(0, pending)
                self.nodes.append(cur)
            else:
                cur.fx_nodes.extend(pending)
            for name in pending:
                self.seg_of[name] = cur.idx
        # 2. users of placeholders and of computed values
        by_name = {n.name: n for n in gm.graph.nodes}
        consumers: Dict[str, Set[int]] = {}
        output_node = next(n for n in gm.graph.nodes if n.op == "output")
        for n in compute:
            seg = self.seg_of[n.name]
            for a in n.all_input_nodes:
                if a.op == "placeholder":
                    info = ph_index[a.name]
                    if info.is_state:
                        self.param_set.users.setdefault(info.index, [])
                        if seg not in self.param_set.users[info.index]:
                            self.param_set.users[info.index].append(seg)
                    else:
                        self.input_users.setdefault(info.index, [])
                        if seg not in self.input_users[info.index]:
                            self.input_users[info.index].append(seg)
                        if info.index not in self.placeholder_order:
                            self.placeholder_order.append(info.index)
                else:
                    consumers.setdefault(a.name, set()).add(seg)
        for a in output_node.all_input_nodes:
            if a.op != "placeholder":
                s = self.seg_of[a.name]
                if s not in self.output_segments:
                    self.output_segments.append(s)
        # 3. parameters: accounted to the first segment that touches them
        for ph, segs in self.param_set.users.items():
            first = min(segs)
            self.param_set.first_use[ph] = first
            info = self.captured.inputs[ph]
            nb = info.tensor.numel() * info.tensor.element_size()
            node = self.nodes[first]
            node.param_inputs.append(ph)
            if info.kind == "param":
                node.param_bytes += nb
                node.weight += WEIGHT_MULTIPLIER * nb
            else:
                node.weight += nb
        # 4. edges between segments + default (unprofiled) statistics
        for n in compute:
            seg = self.seg_of[n.name]
            nb = value_bytes(n)
            node = self.nodes[seg]
            if not is_trivial(n):
                node.out_bytes += nb
            ex = n.meta.get("example_value", n.meta.get("val"))
            shapes = [ShapeMeta.of(t) for t in _tensor_leaves(ex)]
            for c in sorted(consumers.get(n.name, ())):
                if c != seg:
                    self.edges.append(CompEdge(seg, c, n.name, nb, shapes))
        for node in self.nodes:
            node.act_mem = node.out_bytes
            node.temp_mem = node.out_bytes

    # ------------------------------------------------------------------ linearisation
    def linear_order(self, mode: str) -> List[int]:
        """A topological order of the segments for ``--linearizer`` (behaviour of
        pfeife/graph/computation_graph.py:193-277).  Runnable segments are grown into chains
        (a segment whose only unfinished producer is the chain's tail joins it); each round runs
        one whole chain: the one with the fewest segments (``short_first``), the most
        (``long_first``), or the one that leaves the least memory alive while it runs
        (``save_mem``: activations of the other candidates + its own transient peak)."""
        n = len(self.nodes)
        if mode in (None, "none") or n < 2:
            return list(range(n))
        if mode not in ("save_mem", "short_first", "long_first"):
            raise ValueError(f"unknown linearizer {mode!r}")
        preds: List[Set[int]] = [set() for _ in range(n)]
        succs: List[Set[int]] = [set() for _ in range(n)]
        for e in self.edges:
            if e.start != e.end:
                preds[e.end].add(e.start)
                succs[e.start].add(e.end)
        done: Set[int] = set()
        order: List[int] = []
        while len(done) < n:
            chains = []
            for i in range(n):
                if i in done or not preds[i] <= done:
                    continue
                chain, cur = [i], i
                while len(succs[cur]) == 1:
                    nxt = next(iter(succs[cur]))
                    if nxt in done or any(p != cur and p not in done for p in preds[nxt]):
                        break
                    chain.append(nxt)
                    cur = nxt
                chains.append(chain)
            chains.sort(key=len)
            if mode == "short_first":
                taken = chains[0]
            elif mode == "long_first":
                taken = chains[-1]
            else:
                cost = []
                for c in chains:
                    act, peak = 0, 0
                    for i in c:
                        peak = max(peak, self.nodes[i].temp_mem + act)
                        act += self.nodes[i].act_mem
                    cost.append((c, act, peak))
                total = sum(a for _, a, _ in cost)
                taken = min(cost, key=lambda t: total - t[1] + t[2])[0]
            for i in taken:
                if i not in done:
                    done.add(i)
                    order.append(i)
        return order

    def linearize(self, mode: str) -> bool:
        """Re-orders the segments by ``linear_order(mode)`` and the FX graph with them (the
        reference's ``traverse_linearize`` + ``redraw_graph``), keeping the statistics each
        segment already carries.  Returns whether anything moved."""
        order = self.linear_order(mode)
        if order == list(range(len(self.nodes))):
            return False
        gm = self.captured.gm
        by_name = {n.name: n for n in gm.graph.nodes}
        placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
        anchor = placeholders[-1] if placeholders else None
        stats = {}
        for new_idx, old_idx in enumerate(order):
            node = self.nodes[old_idx]
            stats[new_idx] = (node.act_mem, node.temp_mem, node.comp_time, node.back_time,
                              node.optim_time)
            for name in node.fx_nodes:
                fx_node = by_name[name]
                if anchor is None:
                    first = next(iter(gm.graph.nodes))
                    if first is not fx_node:
                        first.prepend(fx_node)
                else:
                    anchor.append(fx_node)
                anchor = fx_node
        gm.graph.lint()
        gm.recompile()
        fb = self.fb_ratio
        self.nodes, self.edges, self.param_set = [], [], ParamSet()
        self.seg_of, self.input_users = {}, {}
        self.output_segments, self.placeholder_order = [], []
        self._build()
        if len(self.nodes) == len(order):
            for idx, (act, temp, t, bt, ot) in stats.items():
                nd = self.nodes[idx]
                nd.act_mem, nd.temp_mem, nd.comp_time, nd.back_time, nd.optim_time = \
                    act, temp, t, bt, ot
        self.fb_ratio = fb
        return True

    # ------------------------------------------------------------------ queries
    def __len__(self) -> int:
        return len(self.nodes)

    def total_time(self) -> float:
        return sum(n.comp_time for n in self.nodes)

    def stage_bounds(self, split_points: Sequence[int]) -> List[Tuple[int, int]]:
        """Split points are segment indices at which a new stage begins."""
        pts = [0] + list(split_points) + [len(self.nodes)]
        return [(pts[i], pts[i + 1]) for i in range(len(pts) - 1)]

    def cross_edges(self, bounds: Sequence[Tuple[int, int]]) -> Dict[Tuple[int, int], int]:
        """(producer stage, consumer stage) -> bytes, each value counted once per consumer
        stage."""
        stage_of = [0] * len(self.nodes)
        for s, (lo, hi) in enumerate(bounds):
            for i in range(lo, hi):
                stage_of[i] = s
        seen: Set[Tuple[str, int]] = set()
        out: Dict[Tuple[int, int], int] = {}
        for e in self.edges:
            a, b = stage_of[e.start], stage_of[e.end]
            if a == b or (e.value, b) in seen:
                continue
            seen.add((e.value, b))
            out[(a, b)] = out.get((a, b), 0) + e.weight
        return out

    # ------------------------------------------------------------------ profile cache
    def graph_data(self) -> Dict[str, Any]:
        return {
            "format": FORMAT,
            "nodes": [dict(weight=n.weight, temp_mem=n.temp_mem, act_mem=n.act_mem,
                           comp_time=n.comp_time, back_time=n.back_time,
                           optim_time=n.optim_time) for n in self.nodes],
            "edges": [dict(weight=e.weight, shape=[(s.size, s.dtype, s.nbytes, s.requires_grad)
                                                   for s in e.shape]) for e in self.edges],
            "fb_ratio": self.fb_ratio,
        }

    def save_graph_data(self, path: str) -> None:
        with open(path, "wb") as f:
            pickle.dump(self.graph_data(), f)

    def load_graph_data(self, path: str) -> None:
        with open(path, "rb") as f:
            self.apply_graph_data(pickle.load(f))

    def apply_graph_data(self, data: Any) -> None:
        """Copies profiled statistics (``graph_data()`` of the same model, or a reference-written
        profile) positionally onto this graph."""
        if isinstance(data, dict) and data.get("format") == FORMAT:
            nodes, edges, fb = data["nodes"], data["edges"], data["fb_ratio"]
            get = lambda o, k: o[k]
        else:  # a reference-written dummy CompGraph (read through same-named shim classes)
            nodes, edges, fb = list(data.nodes), list(data.edges), data.fb_ratio
            get = lambda o, k: getattr(o, k, None)
        if len(nodes) != len(self.nodes):
            raise ValueError(f"graph_bench file has {len(nodes)} segments, the captured graph has "
                             f"{len(self.nodes)}: it was made for another model or batch size")
        for mine, theirs in zip(self.nodes, nodes):
            for k in ("weight", "temp_mem", "act_mem", "comp_time", "optim_time"):
                v = get(theirs, k)
                if v is not None:
                    setattr(mine, k, v)
            try:
                mine.back_time = get(theirs, "back_time")
            except (KeyError, AttributeError):
                mine.back_time = None
        if len(edges) == len(self.edges):
            for mine, theirs in zip(self.edges, edges):
                w = get(theirs, "weight")
                if w is not None:
                    mine.weight = w
        self.fb_ratio = float(fb)

    def summary(self) -> str:
        from ..utils import fmem
        fwd = self.total_time()
        return (f"{len(self.nodes)} segments, {len(self.edges)} edges, forward {fwd:.4f} ms, "
                f"backward {fwd * self.fb_ratio:.4f} ms, params "
                f"{fmem(sum(n.param_bytes for n in self.nodes))}")


def read_comp_graph(captured: CapturedGraph) -> CompGraph:
    return CompGraph(captured)
