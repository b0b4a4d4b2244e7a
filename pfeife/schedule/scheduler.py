from pfeife_b200.parallel.schedule import *  # noqa: F401,F403
from pfeife_b200.parallel.schedule import (BeamScheduler, BFSScheduler, DFSScheduler,  # noqa: F401
                                           ForwardOnlyScheduler, NoSkewScheduler, PipelessScheduler,
                                           PipeSchedParams, PipeSchedSet, Scheduler,
                                           SingleCommScheduler, Step, StepWork)
