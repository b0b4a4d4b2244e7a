"""Names of the reference's computation-graph module.  ``CompGraph`` and friends resolve to
this framework's classes; ``DummyNode`` and attribute-bag versions of ``CompNode`` /
``CompEdge`` exist so that ``--graph_bench`` files pickled by the reference (a dummy
``CompGraph`` whose FX nodes were replaced by ``DummyNode(meta={_weight, _shape})``,
pfeife/graph/computation_graph.py:379-468) can be unpickled and read positionally."""
from pfeife_b200.graph.comp_graph import (GRAPH_FETCH_MEM_CAP, CompEdge, CompGraph, CompNode,  # noqa: F401
                                          ParamSet, ShapeMeta, read_comp_graph)


class DummyNode:
    def __init__(self, meta=None, name=""):
        self.meta = meta or {}
        self.name = name
