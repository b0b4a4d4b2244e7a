"""FX partitioner: cuts a captured graph into pipeline-stage ``GraphModule``s.

Stages are contiguous runs of profiled segments, so the cut is a single pass over the graph in
its original order.  Every stage graph takes, in placeholder order, the states (parameters and
buffers, bound from a per-rank table), the user inputs it reads and the cross-stage values it
consumes; it returns the tuple of values later stages (or the model output, consumer ``-1``)
need.  Skip connections are ordinary edges between non-adjacent stages.  A state used by
stages on different ranks is listed in ``shared_states`` and its gradient is summed over those
ranks before the optimizer step.

Behavioural counterpart of pfeife/graph/partition_graph.py:74-564 (``partition_module``,
``split_rank_gm``, ``input_map/output_map``, ``input_shapes/output_shapes``); parameters are
graph inputs here, so nothing is cloned or re-targeted.
"""
from __future__ import annotations

import copy
import operator
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx

from .comp_graph import CompGraph, ShapeMeta, _tensor_leaves

OUTSIDE = -1  # producer id of user inputs, consumer id of model outputs


@dataclass
class StageInput:
    kind: str                      # "state" | "input" | "edge"
    ph_index: int = -1             # state / input: index among the captured graph's placeholders
    src_stage: int = OUTSIDE       # edge: producing stage
    src_output: int = -1           # edge: index into the producer's outputs
    meta: Optional[ShapeMeta] = None
    name: str = ""


@dataclass
class StageOutput:
    value: str                     # FX node name in the original graph
    meta: Optional[ShapeMeta]
    consumers: List[Tuple[int, int]] = field(default_factory=list)  # (stage | -1, input index)


@dataclass
class StageSpec:
    idx: int
    rank: int
    gm: Optional[fx.GraphModule]
    inputs: List[StageInput] = field(default_factory=list)
    outputs: List[StageOutput] = field(default_factory=list)

    def state_indices(self) -> List[int]:
        return [i.ph_index for i in self.inputs if i.kind == "state"]

    def without_module(self) -> "StageSpec":
        return StageSpec(self.idx, self.rank, None, self.inputs, self.outputs)


class _OutRef:
    """Marker inside ``output_spec``: the `out_idx`-th output of stage `stage`."""

    __slots__ = ("stage", "out_idx")

    def __init__(self, stage: int, out_idx: int):
        self.stage, self.out_idx = stage, out_idx

    def __repr__(self) -> str:
        return f"_OutRef({self.stage}, {self.out_idx})"


class _InRef:
    """Marker inside ``output_spec``: a graph input returned as is."""

    __slots__ = ("ph_index",)

    def __init__(self, ph_index: int):
        self.ph_index = ph_index


@dataclass
class PartitionGraph:
    stages: List[StageSpec]
    output_spec: Any                         # pytree of _OutRef / _InRef / constants
    shared_states: Dict[int, List[int]]      # placeholder index -> ranks using it (>1)
    device_cnt: int
    split_points: List[int]

    def stages_of_rank(self, rank: int) -> List[StageSpec]:
        return [s for s in self.stages if s.rank == rank]

    def rank_states(self, rank: int) -> List[int]:
        seen: List[int] = []
        for s in self.stages_of_rank(rank):
            for i in s.state_indices():
                if i not in seen:
                    seen.append(i)
        return seen

    def for_rank(self, rank: int) -> "PartitionGraph":
        """A copy that keeps stage modules only for `rank` (what is shipped to that worker)."""
        stages = [s if s.rank == rank else s.without_module() for s in self.stages]
        return PartitionGraph(stages, self.output_spec, self.shared_states, self.device_cnt,
                              self.split_points)

    def assemble_output(self, stage_outputs: Dict[Tuple[int, int], Any],
                        graph_inputs: Optional[Sequence[Any]] = None) -> Any:
        def fill(x):
            if isinstance(x, _OutRef):
                return stage_outputs[(x.stage, x.out_idx)]
            if isinstance(x, _InRef):
                return graph_inputs[x.ph_index] if graph_inputs is not None else None
            if isinstance(x, tuple):
                return tuple(fill(e) for e in x)
            if isinstance(x, list):
                return [fill(e) for e in x]
            if isinstance(x, dict):
                return {k: fill(v) for k, v in x.items()}
            return x
        return fill(self.output_spec)

    def sink_outputs(self) -> List[Tuple[int, int]]:
        """(stage, output index) pairs that feed the model output, in a fixed order."""
        out: List[Tuple[int, int]] = []
        for s in self.stages:
            for j, o in enumerate(s.outputs):
                if any(c[0] == OUTSIDE for c in o.consumers):
                    out.append((s.idx, j))
        return out


def _meta_of(node: fx.Node) -> Optional[ShapeMeta]:
    ex = node.meta.get("example_value", node.meta.get("val"))
    if torch.is_tensor(ex):
        return ShapeMeta.of(ex)
    return None


def _const_of(node: fx.Node):
    """(True, value) when the node's value is a plain python constant that can be baked into a
    consumer stage instead of being communicated."""
    ex = node.meta.get("example_value", node.meta.get("val"))
    if ex is None or _tensor_leaves(ex):
        return False, None
    try:
        if isinstance(ex, (int, float, bool, str, torch.dtype, torch.device, type(None))):
            return True, ex
        if isinstance(ex, (tuple, list, torch.Size)) and all(isinstance(e, (int, float, bool))
                                                              for e in ex):
            return True, type(ex)(int(e) if isinstance(e, int) else e for e in ex) \
                if not isinstance(ex, torch.Size) else tuple(int(e) for e in ex)
    except Exception:
        pass
    return False, None


_INPLACE_OPERATORS = {operator.iadd, operator.isub, operator.imul, operator.itruediv,
                      operator.ifloordiv, operator.imod, operator.ipow, operator.iand,
                      operator.ior, operator.ixor}
_VIEW_METHODS = {"view", "reshape", "transpose", "permute", "flatten", "unflatten", "squeeze",
                 "unsqueeze", "t", "view_as", "expand", "narrow", "select", "unbind", "chunk",
                 "split", "contiguous", "detach", "__getitem__"}


def _writes_in_place(n: fx.Node) -> bool:
    """True for a node that overwrites its first argument: a method or function whose name ends
    in one underscore (``relu_``, ``add_``), an augmented assignment, ``inplace=True``."""
    if n.kwargs.get("inplace") is True:
        return True
    if n.op == "call_method":
        return n.target.endswith("_") and not n.target.endswith("__")
    if n.op == "call_function":
        if n.target in _INPLACE_OPERATORS:
            return True
        name = getattr(n.target, "__name__", "")
        return name.endswith("_") and not name.endswith("__")
    return False


def _is_view(n: fx.Node) -> bool:
    if n.op == "call_method":
        return n.target in _VIEW_METHODS
    return n.op == "call_function" and n.target is operator.getitem


def _protect_overwritten_inputs(g: fx.Graph, first_compute: Optional[fx.Node],
                                placeholders: Sequence[fx.Node]) -> None:
    """A value that crosses a stage boundary enters the consuming stage as a leaf tensor that
    requires grad, and autograd refuses to overwrite a leaf.  Where the stage does overwrite one
    (directly, or through a view of it) the stage works on a copy instead; everywhere else the
    received buffer is consumed as it is."""
    if first_compute is None:
        return
    for ph in placeholders:
        seen, todo, hit = set(), [ph], False
        while todo and not hit:
            cur = todo.pop()
            for u in cur.users:
                if u in seen:
                    continue
                seen.add(u)
                if _writes_in_place(u) and u.args and u.args[0] is cur:
                    hit = True
                    break
                if _is_view(u):
                    todo.append(u)
        if hit:
            with g.inserting_before(first_compute):
                copy_node = g.call_method("clone", (ph,))
            ph.replace_all_uses_with(copy_node, delete_user_cb=lambda u: u is not copy_node)


def partition_module(cg: CompGraph, split_points: Sequence[int], device_cnt: int
                     ) -> PartitionGraph:
    captured = cg.captured
    gm = captured.gm
    bounds = cg.stage_bounds(split_points)
    n_stage = len(bounds)
    stage_of_seg = [0] * len(cg.nodes)
    for s, (lo, hi) in enumerate(bounds):
        for i in range(lo, hi):
            stage_of_seg[i] = s
    ph_info = {i.node_name: i for i in captured.inputs}

    graphs = [fx.Graph() for _ in range(n_stage)]
    roots = [torch.nn.Module() for _ in range(n_stage)]
    envs: List[Dict[str, fx.Node]] = [{} for _ in range(n_stage)]
    specs = [StageSpec(s, s % device_cnt, None) for s in range(n_stage)]
    # names of placeholders created so far per stage (they must precede compute nodes)
    first_compute: List[Optional[fx.Node]] = [None] * n_stage
    produced_in: Dict[str, int] = {}
    out_index: Dict[Tuple[int, str], int] = {}

    def new_placeholder(stage: int, name: str) -> fx.Node:
        g = graphs[stage]
        anchor = first_compute[stage]
        if anchor is None:
            return g.placeholder(name)
        with g.inserting_before(anchor):
            return g.placeholder(name)

    def export_value(src_stage: int, value: fx.Node) -> int:
        key = (src_stage, value.name)
        if key not in out_index:
            out_index[key] = len(specs[src_stage].outputs)
            specs[src_stage].outputs.append(StageOutput(value.name, _meta_of(value)))
        return out_index[key]

    def resolve(stage: int, a: fx.Node):
        env = envs[stage]
        if a.name in env:
            return env[a.name]
        if a.op == "placeholder":
            info = ph_info[a.name]
            node = new_placeholder(stage, a.name)
            meta = ShapeMeta.of(info.tensor) if torch.is_tensor(info.tensor) else None
            kind = "state" if info.is_state else "input"
            specs[stage].inputs.append(StageInput(kind, info.index, OUTSIDE, -1, meta, a.name))
            env[a.name] = node
            return node
        src = produced_in[a.name]
        assert src < stage, f"value {a.name} used before its stage"
        is_const, const = _const_of(a)
        if is_const:
            return const
        if _meta_of(a) is None:
            raise NotImplementedError(
                f"value {a.name!r} crossing from stage {src} to {stage} is not a tensor "
                "(tuple-valued or opaque); move the split point")
        j = export_value(src, a)
        node = new_placeholder(stage, f"s{src}_{a.name}")
        in_idx = len(specs[stage].inputs)
        specs[stage].inputs.append(StageInput("edge", -1, src, j, _meta_of(a), a.name))
        specs[src].outputs[j].consumers.append((stage, in_idx))
        env[a.name] = node
        return node

    output_node = None
    for n in gm.graph.nodes:
        if n.op == "placeholder":
            continue
        if n.op == "output":
            output_node = n
            continue
        stage = stage_of_seg[cg.seg_of[n.name]]
        produced_in[n.name] = stage
        g = graphs[stage]
        if n.op == "get_attr":
            obj = gm
            for atom in n.target.split("."):
                obj = getattr(obj, atom)
            flat = n.target.replace(".", "_")
            if isinstance(obj, torch.Tensor):
                roots[stage].register_buffer(flat, obj.detach().clone(), persistent=False)
            else:
                setattr(roots[stage], flat, copy.deepcopy(obj))
            new = g.get_attr(flat)
        else:
            args = fx.node.map_arg(n.args, lambda a: resolve(stage, a))
            kwargs = fx.node.map_arg(n.kwargs, lambda a: resolve(stage, a))
            if n.op == "call_module":
                raise NotImplementedError("call_module nodes are not expected in captured graphs")
            new = g.create_node(n.op, n.target, args, kwargs, name=n.name)
        new.meta = dict(n.meta)
        if first_compute[stage] is None:
            first_compute[stage] = new
        envs[stage][n.name] = new

    # model outputs
    def spec_of(x):
        if isinstance(x, fx.Node):
            if x.op == "placeholder":
                return _InRef(ph_info[x.name].index)
            src = produced_in[x.name]
            if src != n_stage - 1:
                # model outputs always leave through the last stage (it lives on the main
                # rank): an earlier stage's value is passed through it as an ordinary edge
                resolve(n_stage - 1, x)
                src = n_stage - 1
            j = export_value(src, x)
            if not any(c[0] == OUTSIDE for c in specs[src].outputs[j].consumers):
                specs[src].outputs[j].consumers.append((OUTSIDE, -1))
            return _OutRef(src, j)
        if isinstance(x, tuple):
            return tuple(spec_of(e) for e in x)
        if isinstance(x, list):
            return [spec_of(e) for e in x]
        if isinstance(x, dict):
            return {k: spec_of(v) for k, v in x.items()}
        return x

    output_spec = spec_of(output_node.args[0])

    by_name = [{n.name: n for n in g.nodes} for g in graphs]
    for s in range(n_stage):
        edge_phs = [envs[s][i.name] for i in specs[s].inputs
                    if i.kind == "edge" and i.name in envs[s]]
        _protect_overwritten_inputs(graphs[s], first_compute[s], edge_phs)
        outs = tuple(envs[s][o.value] for o in specs[s].outputs)
        graphs[s].output(outs)
        graphs[s].lint()
        specs[s].gm = fx.GraphModule(roots[s], graphs[s], class_name=f"Stage{s}")

    shared: Dict[int, List[int]] = {}
    users: Dict[int, List[int]] = {}
    for sp in specs:
        for i in sp.state_indices():
            if captured.inputs[i].kind == "param":
                users.setdefault(i, [])
                if sp.rank not in users[i]:
                    users[i].append(sp.rank)
    for i, ranks in users.items():
        if len(ranks) > 1:
            shared[i] = sorted(ranks)
    return PartitionGraph(specs, output_spec, shared, device_cnt, list(split_points))


def partition_module_by_pgraph(cg: CompGraph, pipe_graph, devices=None) -> PartitionGraph:
    """Spelling of the reference entry point (pfeife/graph/partition_graph.py:545-564)."""
    pts = [n.lo for n in pipe_graph.nodes[1:]]
    return partition_module(cg, pts, pipe_graph.device_cnt)


def check_partition(cg: CompGraph, part: PartitionGraph, args: Sequence[Any]) -> Any:
    """Runs the stages in order on one device and returns the assembled output (tests use this
    to check that the composition of the stages equals the original graph)."""
    produced: Dict[Tuple[int, int], Any] = {}
    for sp in part.stages:
        ins = []
        for i in sp.inputs:
            if i.kind in ("state", "input"):
                ins.append(args[i.ph_index])
            else:
                ins.append(produced[(i.src_stage, i.src_output)])
        outs = sp.gm(*ins)
        for j, o in enumerate(outs):
            produced[(sp.idx, j)] = o
    return part.assemble_output(produced, args)
