from pfeife_b200.runtime.partial import (STEP_TOKEN, PartialModule, PartialRunner,  # noqa: F401
                                         partial_compiler)
