from pfeife_b200.topology import *  # noqa: F401,F403
from pfeife_b200.topology import (PfeifeState, check_main_rank, get_device, get_dp_group_ranks,  # noqa: F401
                                  get_global_rank, get_pp_group_ranks, get_pp_rank, get_state,
                                  initialize_pfeife, parse_dp_mesh, target_main_rank)
