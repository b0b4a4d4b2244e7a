from pfeife_b200.parallel.planner import *  # noqa: F401,F403
from pfeife_b200.parallel.planner import (BeamSearchGenerator, BeamSingleGenerator,  # noqa: F401
                                          DependencyGraph, PipeGraphGenerator, SchedCommNode,
                                          SchedCompNode, SchedNode, choose_mesh, get_pipe_class)
