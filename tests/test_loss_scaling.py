"""Dynamic loss scaling on the host path (the device path runs the same rules in kernels and is
covered by the GPU training tests): a non-finite gradient skips the update and halves the scale,
a run of clean steps doubles it."""
import torch

from pfeife_b200.runtime.params import LossScaler, RankParams, StateEntry


def _params():
    entries = [StateEntry(0, "w", "param", torch.ones(4, 4), True, 0),
               StateEntry(1, "b", "param", torch.zeros(4), True, 0)]
    return RankParams(entries, torch.device("cpu"), None, "sgd", [{"lr": 0.5}], native=False)


def test_non_finite_gradient_skips_the_step_and_backs_the_scale_off():
    p = _params()
    scaler = LossScaler(torch.device("cpu"), True, init_scale=1024.0, growth_interval=2)
    w0 = p.slots[0].master.clone()
    p.slots[0].grad.fill_(1.0)
    p.slots[1].grad[0] = float("inf")
    p.check_finite()
    assert float(p.found_inf) == 1.0
    p.step(loss_scale=scaler.scale_tensor, use_found_inf=True)
    scaler.update(p.found_inf)
    assert torch.equal(p.slots[0].master, w0)            # update skipped
    assert float(p.grad.abs().sum()) == 0.0               # gradients consumed all the same
    assert scaler.get_scale() == 512.0 and float(p.found_inf) == 0.0


def test_clean_steps_unscale_the_gradient_and_grow_the_scale():
    p = _params()
    scaler = LossScaler(torch.device("cpu"), True, init_scale=8.0, growth_interval=2)
    for i in range(2):
        w0 = p.slots[0].master.clone()
        p.slots[0].grad.fill_(8.0 * scaler.get_scale() / 8.0)   # a true gradient of 1, scaled
        p.check_finite()
        p.step(loss_scale=scaler.scale_tensor, use_found_inf=True)
        scaler.update(p.found_inf)
        assert torch.allclose(p.slots[0].master, w0 - 0.5)      # lr 0.5 x unscaled gradient 1
    assert scaler.get_scale() == 16.0                            # two clean steps: doubled


def test_disabled_scaler_is_the_identity():
    scaler = LossScaler(torch.device("cpu"), False)
    loss = torch.tensor(3.0)
    assert scaler.scale(loss) is loss and scaler.scale_tensor is None
    scaler.update(torch.zeros(1))
    assert scaler.get_scale() == 1.0
