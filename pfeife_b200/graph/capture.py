"""Graph capture for current PyTorch (>= 2.4): the dynamo backend receives a flat graph of
``placeholder / call_function / call_method / output`` nodes in which parameters and buffers
arrive as graph inputs (``example_inputs`` holds the model's real ``nn.Parameter`` objects and
``node.meta['grapharg'].source.name`` spells ``L['self']._modules['blocks']...``).

This module classifies the placeholders and builds the parameter table
``placeholder -> (qualified name, tensor)``.  Tied weights show up as ONE placeholder with
several users, so no clone bookkeeping is needed (the reference clones re-used modules,
pfeife/graph/computation_graph.py:701-754, because its torch-2.3 graphs carry ``call_module``
nodes).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence

import torch
import torch.fx as fx

_SRC_ATOM = re.compile(r"\._(modules|parameters|buffers)\['([^']+)'\]|\.([A-Za-z_][A-Za-z_0-9]*)")


def qualified_name(source_name: Optional[str], fallback: str) -> str:
    """"L['self']._modules['blocks']._modules['0']._parameters['weight']" -> "blocks.0.weight"."""
    if not source_name:
        return fallback
    rest = source_name
    m = re.match(r"^[LG]\['[^']+'\]", rest)
    if m:
        rest = rest[m.end():]
    atoms = []
    for kind, key, attr in _SRC_ATOM.findall(rest):
        atoms.append(key if key else attr)
    return ".".join(atoms) if atoms else fallback


@dataclass
class GraphInput:
    index: int               # position among the graph's placeholders
    node_name: str
    kind: str                # "param" | "buffer" | "input"
    qualname: str
    tensor: Any              # the real Parameter / buffer (params, buffers) or the example input
    requires_grad: bool = False

    @property
    def is_state(self) -> bool:
        return self.kind in ("param", "buffer")


@dataclass
class CapturedGraph:
    gm: fx.GraphModule
    inputs: List[GraphInput]

    @property
    def params(self) -> List[GraphInput]:
        return [i for i in self.inputs if i.kind == "param"]

    @property
    def buffers(self) -> List[GraphInput]:
        return [i for i in self.inputs if i.kind == "buffer"]

    @property
    def user_inputs(self) -> List[GraphInput]:
        return [i for i in self.inputs if i.kind == "input"]

    def compute_node_count(self) -> int:
        return sum(1 for n in self.gm.graph.nodes if n.op in ("call_function", "call_method",
                                                                "call_module"))

    def shadow_only_inputs(self) -> set:
        """Indices of the state placeholders that are read ONLY as the weight operand of the
        native GEMM-like ops (linear, fused MLP, convolution, embedding).  Under mixed precision
        those ops read the 16-bit shadow of the weight, never its fp32 master, so a
        data-parallel rank that does not own such a parameter needs no current master copy of
        it.  Anything else (biases, norm weights, position embeddings, a weight that an ATen op
        touches) is read in fp32."""
        out = set()
        by_name = {n.name: n for n in self.gm.graph.nodes}
        for gi in self.inputs:
            if not gi.is_state:
                continue
            node = by_name.get(gi.node_name)
            users = list(node.users) if node is not None else []
            if users and all(_reads_shadow(u, node) for u in users):
                out.add(gi.index)
        return out

    def split_call_args(self, args: Sequence[Any]) -> List[Any]:
        """Runtime call arguments (in placeholder order) -> just the user inputs."""
        return [args[i.index] for i in self.inputs if i.kind == "input"]


# op name -> positions of the weight operands that the op reads through the 16-bit shadow
_SHADOW_OPERANDS = {"linear_fwd": (1,), "mlp_fwd": (1, 3), "conv2d_fwd": (1,), "embed_fwd": (1,)}


def _reads_shadow(user: fx.Node, value: fx.Node) -> bool:
    if user.op != "call_function":
        return False
    name = str(user.target)
    if "pfeife" not in name:
        return False
    for op, positions in _SHADOW_OPERANDS.items():
        if f"pfeife.{op}" in name or f"pfeife::{op}" in name:
            uses = [i for i, a in enumerate(user.args) if a is value]
            return bool(uses) and all(i in positions for i in uses) and \
                value not in user.kwargs.values()
    return False


def _source_name(node: fx.Node) -> Optional[str]:
    ga = node.meta.get("grapharg")
    src = getattr(ga, "source", None) if ga is not None else None
    if src is None:
        return None
    name = getattr(src, "name", None)
    if callable(name):
        try:
            name = name()
        except Exception:
            name = None
    return name


def classify_inputs(gm: fx.GraphModule, example_inputs: Sequence[Any]) -> CapturedGraph:
    placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
    if len(placeholders) != len(example_inputs):
        raise RuntimeError("placeholder / example input count mismatch")
    # graphs from older stacks (or hand-written GraphModules) may still own parameters
    owned = dict(gm.named_parameters())
    inputs: List[GraphInput] = []
    for i, (node, ex) in enumerate(zip(placeholders, example_inputs)):
        src = _source_name(node)
        if isinstance(ex, torch.nn.Parameter) or (src and "_parameters[" in src):
            kind = "param"
        elif torch.is_tensor(ex) and src and "_buffers[" in src:
            kind = "buffer"
        else:
            kind = "input"
        inputs.append(GraphInput(i, node.name, kind, qualified_name(src, node.name), ex,
                                 bool(torch.is_tensor(ex) and ex.requires_grad)))
    if owned:
        raise RuntimeError(
            "the captured GraphModule owns parameters (call_module graph); this framework "
            "expects parameters as graph inputs (torch >= 2.4 with inline_inbuilt_nn_modules)")
    return CapturedGraph(gm, inputs)
