"""Loss wrappers with the ``(input, target, model)`` call shape used by the manager-style APIs
and the benchmarks (pfeife/loss.py:4-70)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class LossWrapper(nn.Module):
    """Base of the wrappers; on its own it sums the output, like the reference's base class."""

    def forward(self, input, target=None, model=None):
        return _first_tensor(input).float().sum()


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
    """Uses the ``loss`` field a HuggingFace head already computed; a head that was given no
    labels leaves it ``None``, and the sum of the logits stands in."""

    def forward(self, input, target=None, model=None):
        loss = getattr(input, "loss", None)
        if loss is None and isinstance(input, dict):
            loss = input.get("loss")
        if loss is not None:
            return loss
        return _first_tensor(input).float().sum()


class RescaleLoss(LossWrapper):
    def __init__(self, loss_fn, scale: float = 1.0):
        super().__init__()
        self.loss_fn, self.scale = loss_fn, scale

    def forward(self, input, target, model=None):
        return self.loss_fn(input, target, model) * self.scale


class NormalizeLoss(LossWrapper):
    """Scales the wrapped loss by the power of two that brings its magnitude into (0.5, 1]; a
    zero loss passes through.  The reference finds the factor with ``.item()`` in two host loops
    (doubling while below 1, halving while above 1); here the exponent is read off the value on
    the device with ``frexp``, so the step needs no host sync and can sit inside a CUDA graph."""

    def __init__(self, loss_fn):
        super().__init__()
        self.loss_fn = loss_fn

    def forward(self, input, target, model=None):
        loss = self.loss_fn(input, target, model)
        mant, exp = torch.frexp(loss.detach().float())
        # |loss| = mant * 2^exp with mant in [0.5, 1): dividing by 2^exp lands in [0.5, 1); an exact
        # power of two (mant == 0.5) ends the reference's loops at 1, one doubling further
        exp = exp - (mant.abs() == 0.5).to(exp.dtype)
        return loss * torch.ldexp(torch.ones_like(mant), -exp).to(loss.dtype)


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
