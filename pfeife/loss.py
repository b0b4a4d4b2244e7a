from pfeife_b200.loss import *  # noqa: F401,F403
from pfeife_b200.loss import (CrossEntropyLoss, HFCrossEntropyLoss, LossWrapper,  # noqa: F401
                              MaskedLMOutputLoss, NormalizeLoss, RescaleLoss, SumLoss)
