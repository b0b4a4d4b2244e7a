"""Capture, segmentation, profile cache and partitioning on CPU: the composition of the stage
graphs must equal the original graph for every split, including skip connections, tied weights
and multi-output models."""
import itertools
import os

import pytest
import torch

from pfeife_b200.graph.capture import classify_inputs, qualified_name
from pfeife_b200.graph.comp_graph import CompGraph
from pfeife_b200.graph.partition import check_partition, partition_module
from pfeife_b200.graph.profiler import gen_comp_graph_cpu, gen_local_comp_graph
from pfeife_b200.models.toy import DeepMLP, SkipNet, TiedMLP
from pfeife_b200.models.vit import ViT, vit_config
from pfeife_b200.option import PipeOption


def capture(model, *args, **kwargs):
    box = {}

    def backend(gm, example_inputs):
        box["cap"] = classify_inputs(gm, example_inputs)
        box["args"] = list(example_inputs)
        return gm.forward

    torch._dynamo.reset()
    out = torch.compile(model, backend=backend)(*args, **kwargs)
    return box["cap"], box["args"], out


def test_qualified_name():
    assert qualified_name("L['self']._modules['blocks']._modules['0']._parameters['weight']",
                          "x") == "blocks.0.weight"
    assert qualified_name("L['s']._buffers['pos']", "x") == "pos"
    assert qualified_name(None, "fallback") == "fallback"


def test_capture_classifies_params_buffers_inputs():
    model = ViT(vit_config("vit_tiny", num_layers=2, image_size=32, patch_size=16))
    cap, args, out = capture(model, torch.randn(2, 3, 32, 32))
    names = {i.qualname for i in cap.params}
    assert names == {n for n, _ in model.named_parameters()}
    assert len(cap.user_inputs) == 1 and cap.user_inputs[0].tensor.shape == (2, 3, 32, 32)
    # the table holds the model's own Parameter objects
    by_name = dict(model.named_parameters())
    assert all(i.tensor is by_name[i.qualname] for i in cap.params)


def test_tied_weight_is_one_placeholder():
    cap, _, _ = capture(TiedMLP(), torch.randn(4, 10))
    assert len(cap.params) == 2 + 2   # first(=last) weight/bias + middle weight/bias
    cg = CompGraph(cap)
    shared = [ph for ph, segs in cg.param_set.users.items() if len(segs) > 1]
    assert len(shared) == 2


@pytest.mark.parametrize("model_fn,inp", [
    (lambda: DeepMLP(16, 6, 4), (5, 16)),
    (lambda: SkipNet(16, 3), (5, 16)),
    (lambda: TiedMLP(10, 2), (5, 10)),
])
def test_partition_composition_equals_original(model_fn, inp):
    torch.manual_seed(0)
    model = model_fn()
    x = torch.randn(*inp)
    cap, args, ref = capture(model, x)
    cg = CompGraph(cap)
    n = len(cg.nodes)
    assert n >= 4
    for k in (1, 2, 3):
        for pts in itertools.islice(itertools.combinations(range(1, n), k), 0, 40, 7):
            part = partition_module(cg, list(pts), device_cnt=2)
            assert len(part.stages) == k + 1
            out = check_partition(cg, part, args)
            got = out[0] if isinstance(out, (tuple, list)) else out
            assert torch.allclose(got, ref, atol=1e-6), pts


def test_partition_vit_with_native_ops_and_shared_detection():
    torch.manual_seed(0)
    model = ViT(vit_config("vit_tiny", num_layers=3, image_size=32, patch_size=16))
    x = torch.randn(2, 3, 32, 32)
    cap, args, ref = capture(model, x)
    cg = CompGraph(cap)
    n = len(cg.nodes)
    part = partition_module(cg, [n // 3, 2 * n // 3], device_cnt=3)
    out = check_partition(cg, part, args)
    assert torch.allclose(out[0], ref, atol=1e-5)
    assert part.shared_states == {}
    # every parameter is owned by exactly one rank
    owned = [i for r in range(3) for i in part.rank_states(r)]
    assert sorted(set(owned)) == sorted(i.index for i in cap.inputs if i.is_state)
    # gradients flow through the partitioned graph like through the original
    ref.sum().backward()
    g_ref = {n_: p.grad.clone() for n_, p in model.named_parameters()}
    model.zero_grad()
    check_partition(cg, part, args)[0].sum().backward()
    for n_, p in model.named_parameters():
        assert torch.allclose(p.grad, g_ref[n_], atol=1e-5), n_


def test_tied_params_across_ranks_are_reported_shared():
    cap, args, ref = capture(TiedMLP(10, 2), torch.randn(4, 10))
    cg = CompGraph(cap)
    part = partition_module(cg, [len(cg.nodes) // 2], device_cnt=2)
    assert len(part.shared_states) == 2
    assert all(r == [0, 1] for r in part.shared_states.values())


def test_multi_output_dict_model():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(8, 8)
            self.b = torch.nn.Linear(8, 4)

        def forward(self, x):
            h = torch.relu(self.a(x))
            return {"hidden": h, "logits": self.b(h), "const": 3}

    cap, args, ref = capture(M(), torch.randn(3, 8))
    cg = CompGraph(cap)
    part = partition_module(cg, [2], device_cnt=2)
    out = check_partition(cg, part, args)
    assert len(part.sink_outputs()) == 2


def test_graph_bench_cache_roundtrip(tmp_path):
    cap, args, _ = capture(DeepMLP(16, 4, 4), torch.randn(5, 16))
    path = str(tmp_path / "toy.graph")
    opt = PipeOption(device_cnt=2, graph_bench=path, no_bench_optimizer=True, cpu_test=True)
    cg, out = gen_local_comp_graph(cap, args, torch.device("cpu"), opt)
    assert os.path.exists(path) and all(n.comp_time > 0 for n in cg.nodes)
    cg2, _ = gen_local_comp_graph(cap, args, torch.device("cpu"), opt)   # loads the cache
    assert [n.comp_time for n in cg2.nodes] == [n.comp_time for n in cg.nodes]
    assert cg2.fb_ratio == cg.fb_ratio
    cgu, _ = gen_comp_graph_cpu(cap, args, opt)
    assert all(n.comp_time == 1.0 for n in cgu.nodes) and cgu.fb_ratio == 2.0


class _Branchy(torch.nn.Module):
    def __init__(self):
        super().__init__()
        mk = lambda: torch.nn.Linear(8, 8)
        self.a, self.b1, self.b2, self.c1, self.d = mk(), mk(), mk(), mk(), mk()

    def forward(self, x):
        h = self.a(x)
        long = torch.relu(self.b2(torch.relu(self.b1(h))))
        short = self.c1(h)
        return self.d(long + short)


@pytest.mark.parametrize("mode", ["save_mem", "short_first", "long_first"])
def test_linearizers_keep_the_function_and_order_the_branches(mode):
    """--linearizer: a topological re-ordering of the segments (and of the FX graph with them):
    the short branch runs first under ``short_first``, the long one under ``long_first``, and
    the graph computes the same function either way."""
    torch.manual_seed(0)
    model = _Branchy()
    x = torch.randn(3, 8)
    cap, args, ref = capture(model, x)
    cg = CompGraph(cap)
    n = len(cg.nodes)
    order = cg.linear_order(mode)
    assert sorted(order) == list(range(n))
    pos = {seg: i for i, seg in enumerate(order)}
    for e in cg.edges:                      # producers stay ahead of their consumers
        assert pos[e.start] < pos[e.end]
    names_before = [nd.fx_nodes[-1] for nd in cg.nodes]
    moved = cg.linearize(mode)
    names_after = [nd.fx_nodes[-1] for nd in cg.nodes]
    assert sorted(names_before) == sorted(names_after)
    if mode == "short_first":
        assert moved and names_after.index("short") < names_after.index("long")
    if mode == "long_first":
        assert names_after.index("long") < names_after.index("short")
    part = partition_module(cg, [n // 2], device_cnt=2)
    out = check_partition(cg, part, args)
    got = out[0] if isinstance(out, (tuple, list)) else out
    assert torch.allclose(got, ref, atol=1e-6)


def test_linearizer_option_reaches_the_profile():
    cap, args, ref = capture(_Branchy(), torch.randn(3, 8))
    opt = PipeOption(device_cnt=2, linearizer="short_first", no_bench_optimizer=True, cpu_test=True)
    cg, out = gen_comp_graph_cpu(cap, args, opt)
    names = [nd.fx_nodes[-1] for nd in cg.nodes]
    assert names.index("short") < names.index("long")


def test_compile_hook_wraps_a_stage_module():
    """--backend: a stage module is compiled with the named dynamo backend on first use
    (pfeife/compile.py:19-60); no backend leaves the module as it is."""
    from pfeife_b200.compile import WrapperModule, compile_module
    mod = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU())
    assert compile_module(None, mod) is mod
    wrapped = compile_module("eager", mod)
    assert isinstance(wrapped, WrapperModule)
    x = torch.randn(2, 4)
    assert torch.allclose(wrapped(x), mod(x))
    single = WrapperModule(lambda *a: (a[0] * 2,), unwrap_singleton_tuple=True)
    assert torch.equal(single(x), x * 2)


def test_optimizer_timing_leaves_the_probing_graph_usable():
    """The optimizer is timed while the probing forward's autograd graph is still alive (its
    backward runs afterwards, in the caller): the real parameters must keep their values and
    their version counters, so the measurement steps stand-ins."""
    model = DeepMLP(16, 4, 4)
    cap, args, _ = capture(model, torch.randn(5, 16))
    opt = PipeOption(device_cnt=2, cpu_test=True, optimizer={"type": "adam", "lr": 0.1})
    before = [(p.detach().clone(), p._version) for p in model.parameters()]
    cg, out = gen_local_comp_graph(cap, args, torch.device("cpu"), opt)
    assert sum(n.optim_time for n in cg.nodes) > 0.0        # the optimizer was measured
    for p, (val, ver) in zip(model.parameters(), before):
        assert p._version == ver and torch.equal(p.detach(), val) and p.grad is None
    first = out[0] if isinstance(out, (tuple, list)) else out
    first.sum().backward()                                   # the caller's backward still works
    assert all(p.grad is not None for p in model.parameters())


def test_declared_stage_precision_reaches_the_trace():
    """Meta functions of a trace run with autocast off.  With the stages' precision declared,
    the linear op reports the 16-bit output it will really produce, and a ``.to(y.dtype)`` of
    the model is baked into the graph with that type (it was float32 before, and the stages
    then mixed fp32 and 16-bit tensors)."""
    from pfeife_b200 import ops
    from pfeife_b200.ops import functional as Fn
    w, b = torch.randn(8, 8), torch.zeros(8)

    def f(x):
        y = ops.linear(x, w, b)
        return y + torch.ones(8).to(y.dtype)

    def trace(declared):
        box = {}

        def backend(gm, example_inputs):
            box["code"] = gm.code
            return gm.forward

        torch._dynamo.reset()
        with Fn.stage_precision(declared), torch.autocast("cpu", torch.bfloat16,
                                                          enabled=declared is not None):
            out = torch.compile(f, backend=backend)(torch.randn(4, 8))
        return box["code"], out

    code, out = trace(torch.bfloat16)
    assert "torch.bfloat16" in code and "torch.float32" not in code
    assert out.dtype == torch.bfloat16
    code, out = trace(None)
    assert "torch.bfloat16" not in code and out.dtype == torch.float32


def test_backward_times_are_per_segment_and_keep_the_total():
    """Every segment gets a backward time of its own (proportions of one eager backward), and
    the times add up to the backward total the planner used before (ratio x forward total)."""
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 64)
            self.big = torch.nn.Linear(64, 4096)
            self.big2 = torch.nn.Linear(4096, 64)
            self.c = torch.nn.Linear(64, 8)

        def forward(self, x):
            h = torch.relu(self.a(x))
            h = torch.relu(self.big2(torch.relu(self.big(h))))
            return self.c(h)

    torch.manual_seed(0)
    cap, args, _ = capture(Net(), torch.randn(512, 64))
    opt = PipeOption(device_cnt=2, no_bench_optimizer=True, cpu_test=True)
    cg, _ = gen_local_comp_graph(cap, args, torch.device("cpu"), opt)
    back = [n.back_time for n in cg.nodes]
    assert all(b is not None and b > 0 for b in back)
    fwd_total = sum(n.comp_time for n in cg.nodes)
    assert sum(back) == pytest.approx(cg.fb_ratio * fwd_total, rel=1e-3)
    # the two wide layers dominate the backward as they dominate the forward
    wide = sorted(range(len(back)), key=lambda i: -back[i])[:3]
    heavy_fwd = sorted(range(len(back)), key=lambda i: -cg.nodes[i].comp_time)[:3]
    assert set(wide) & set(heavy_fwd)
    ratios = [b / n.comp_time for b, n in zip(back, cg.nodes)]
    assert max(ratios) > 1.5 * min(ratios)          # not one ratio for all
