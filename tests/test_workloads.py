"""Benchmark workloads: every named configuration builds (the big ones on the meta device, to
check shapes and parameter counts) and the reduced ones train a step's worth of loss on CPU."""
import pytest
import torch

from pfeife_b200.bench.workloads import WORKLOADS, get_workload


@pytest.mark.parametrize("name", ["vit_tiny", "llama_tiny", "unet_tiny"])
def test_reduced_workloads_produce_a_finite_loss_and_gradients(name):
    wl = get_workload(name)
    torch.manual_seed(0)
    model = wl.build_model()
    batch = wl.make_batch(wl.micro_batch, torch.Generator().manual_seed(1))
    assert len(batch) >= wl.n_model_inputs
    loss = wl.loss(model, *batch)
    assert loss.dim() == 0 and torch.isfinite(loss)
    loss.backward()
    assert any(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize("name,params_b,mesh", [
    ("vitg", 1.01, None), ("vitl", 0.30, "-2,4"), ("llama7b", 6.74, "8"),
    ("llama7b_fsdp", 6.74, "-2,4"), ("sdxl", 2.57, "2,-4")])
def test_full_size_workloads_have_the_named_shapes(name, params_b, mesh):
    wl = get_workload(name)
    assert name in WORKLOADS and wl.mesh_for_8 == mesh
    with torch.device("meta"):
        model = wl.build_model()
    n = sum(p.numel() for p in model.parameters()) / 1e9
    assert n == pytest.approx(params_b, rel=0.03), n
    if name == "llama7b":
        assert wl.option == {"loop_cnt": 2} and wl.micro_batch == 1 and wl.batch_cnt == 16
    if name == "llama7b_fsdp":
        assert wl.option == {"use_fsdp": True}
    if name == "vitl":
        assert wl.option == {"prefetch_fwd": 2} and wl.micro_batch == 16
