"""Loss wrappers against plain PyTorch and against the rules of the reference's wrappers
(pfeife/loss.py:4-70)."""
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from pfeife_b200.loss import (CrossEntropyLoss, HFCrossEntropyLoss, LossWrapper, MaskedLMOutputLoss,
                              NormalizeLoss, RescaleLoss, SumLoss, _first_tensor)


def test_first_tensor_finds_the_leading_tensor():
    t = torch.ones(2, 3)
    assert _first_tensor(t) is t
    assert _first_tensor((t, None)) is t
    assert _first_tensor([[t], 3]) is t
    assert _first_tensor({"a": t, "b": 1}) is t
    assert _first_tensor(SimpleNamespace(logits=t)) is t
    with pytest.raises(TypeError):
        _first_tensor(3)


def test_base_and_sum_loss():
    x = torch.randn(4, 5, requires_grad=True)
    for fn in (LossWrapper(), SumLoss()):
        x.grad = None
        loss = fn((x, "other"), None)
        assert torch.allclose(loss, x.sum())
        loss.backward()
        assert torch.equal(x.grad, torch.ones_like(x))
    half = torch.randn(4, 5).half()
    assert SumLoss()(half, None).dtype == torch.float32


def test_masked_lm_output_loss():
    logits = torch.randn(2, 3)
    out = SimpleNamespace(loss=torch.tensor(1.25), logits=logits)
    assert float(MaskedLMOutputLoss()(out, None)) == 1.25
    out = SimpleNamespace(loss=None, logits=logits)
    assert torch.allclose(MaskedLMOutputLoss()(out, None), logits.sum())
    assert float(MaskedLMOutputLoss()({"loss": torch.tensor(2.0), "logits": logits}, None)) == 2.0


def test_rescale_loss():
    x = torch.randn(3, 3)
    assert torch.allclose(RescaleLoss(SumLoss(), 0.25)(x, None), x.sum() * 0.25)


def _reference_normalize(v: float) -> float:
    if v == 0:
        return v
    while abs(v) < 1:
        v *= 2
    while abs(v) > 1:
        v /= 2
    return v


@pytest.mark.parametrize("value", [0.0, 1.0, -1.0, 0.5, 2.0, 1024.0, 3.7, -3.7, 1e-4, -0.3, 777.0, 0.999])
def test_normalize_loss_matches_the_doubling_rule(value):
    x = torch.tensor([value], requires_grad=True)
    loss = NormalizeLoss(SumLoss())(x, None)
    want = _reference_normalize(float(torch.tensor(value)))
    assert float(loss) == pytest.approx(want, rel=1e-6)
    if value != 0:
        assert 0.5 < abs(float(loss)) <= 1.0
        loss.backward()
        # the factor is a constant of the graph: d loss / d x is the factor itself
        assert float(x.grad) == pytest.approx(want / value, rel=1e-6)


def test_cross_entropy_wrappers():
    logits = torch.randn(2, 7, 10)
    target = torch.randint(0, 10, (2, 7))
    want = F.cross_entropy(logits.view(-1, 10), target.view(-1))
    assert torch.allclose(CrossEntropyLoss(10)(logits, target.view(-1)), want)
    assert torch.allclose(CrossEntropyLoss(10)(logits, target), want)
    assert torch.allclose(HFCrossEntropyLoss(10)(SimpleNamespace(logits=logits), target), want)
    # half logits are upcast before the softmax
    got = CrossEntropyLoss(10)(logits.half(), target)
    assert got.dtype == torch.float32 and torch.allclose(got, want, atol=5e-3)
