from pfeife_b200.parallel.pipe_graph import PipeEdge, PipeGraph, PipeNode  # noqa: F401
