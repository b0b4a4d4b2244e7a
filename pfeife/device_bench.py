from pfeife_b200.parallel.device_bench import *  # noqa: F401,F403
from pfeife_b200.parallel.device_bench import (DeviceBench, NCCLDeviceBench, biased_relu,  # noqa: F401
                                               fit_link, main)
