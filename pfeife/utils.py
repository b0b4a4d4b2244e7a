from pfeife_b200.utils import *  # noqa: F401,F403
from pfeife_b200.utils import (MinMaxRecorder, Recorder, fetch_attr, fmem, get_logger,  # noqa: F401
                               get_submodules, list_params, module_set_attr, set_logger_level,
                               set_seed, to_device, to_device_graphmodule, tree_filter,
                               tree_filter_tensor, tree_trav)
