from pfeife_b200.option import *  # noqa: F401,F403
from pfeife_b200.option import PipeOption, default_optimizer, get_optimizer_cls  # noqa: F401
