from pfeife_b200.graph.partition import (PartitionGraph, StageSpec, partition_module,  # noqa: F401
                                         partition_module_by_pgraph)
