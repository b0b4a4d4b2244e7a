from pfeife_b200.graph.profiler import (TIME_CHECK_ITER, TIME_WARM_ITER, gen_amp_context,  # noqa: F401
                                        gen_comp_graph_cpu, gen_local_comp_graph,
                                        measure_optimizer)

gen_comp_graph = gen_local_comp_graph
