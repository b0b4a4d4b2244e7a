from pfeife_b200.utils.batch import *  # noqa: F401,F403
from pfeife_b200.utils.batch import send_value, shard_dict_of_args, split_args_kwargs  # noqa: F401
