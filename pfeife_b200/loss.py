"""Loss wrappers with the ``(input, target, model)`` call shape used by the manager-style APIs
and the benchmarks (pfeife/loss.py:4-70)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class LossWrapper(nn.Module):
    def forward(self, input, target, model=None):
        raise NotImplementedError


def _first_tensor(out):
    if torch.is_tensor(out):
        return out
    if hasattr(out, "logits"):
        return out.logits
    if isinstance(out, (tuple, list)):
        return _first_tensor(out[0])
    if isinstance(out, dict):
        return _first_tensor(next(iter(out.values())))
    raise TypeError(f"cannot find a tensor in {type(out)}")


class SumLoss(LossWrapper):
    """Sum of every element of the (first) output: a loss with a trivially known gradient."""

    def forward(self, input, target=None, model=None):
        return _first_tensor(input).float().sum()


class MaskedLMOutputLoss(LossWrapper):
    """Uses the ``loss`` field a HuggingFace head already computed."""

    def forward(self, input, target=None, model=None):
        return input.loss if hasattr(input, "loss") else input[0]


class RescaleLoss(LossWrapper):
    def __init__(self, loss_fn, scale: float = 1.0):
        super().__init__()
        self.loss_fn, self.scale = loss_fn, scale

    def forward(self, input, target, model=None):
        return self.loss_fn(input, target, model) * self.scale


class NormalizeLoss(LossWrapper):
    """Divides the wrapped loss by the number of elements of the output."""

    def __init__(self, loss_fn):
        super().__init__()
        self.loss_fn = loss_fn

    def forward(self, input, target, model=None):
        return self.loss_fn(input, target, model) / max(1, _first_tensor(input).numel())


class CrossEntropyLoss(LossWrapper):
    def __init__(self, num_labels: int = 10):
        super().__init__()
        self.num_labels = num_labels

    def forward(self, input, target, model=None):
        logits = _first_tensor(input)
        return F.cross_entropy(logits.reshape(-1, self.num_labels).float(), target.reshape(-1))


class HFCrossEntropyLoss(CrossEntropyLoss):
    """Cross entropy on the ``logits`` field of a HuggingFace output object."""

    def forward(self, input, target, model=None):
        logits = input.logits if hasattr(input, "logits") else _first_tensor(input)
        return F.cross_entropy(logits.reshape(-1, self.num_labels).float(), target.reshape(-1))
