"""Schedules, cost model and planner on synthetic graphs (pure CPU)."""
import itertools
import random

import pytest
import torch

from pfeife_b200.option import PipeOption
from pfeife_b200.parallel import schedule as S
from pfeife_b200.parallel.device_bench import DeviceBench, fit_link, nvswitch_default
from pfeife_b200.parallel.pipe_graph import PipeEdge, PipeGraph, PipeNode
from pfeife_b200.parallel.planner import (BeamSingleGenerator, build_pipe_graph, choose_mesh,
                                          dp_exposed_time, get_pipe_class)
from pfeife_b200.topology import MeshLayout, check_main_rank, parse_dp_mesh


def fmt(p):
    return [" ".join(f"{s}{'F' if f else 'B'}{b}" for s, b, f in w) for w in p.rank_works]


GOLDEN = {
    (2, 4, 2, 4, 0): ["0F0 0F1 0B0 0F2 0B1 0F3 0B2 0B3", "1F0 1B0 1F1 1B1 1F2 1B2 1F3 1B3"],
    (2, 4, 2, 4, 1): ["0F0 0F1 0F2 0B0 0F3 0B1 0B2 0B3", "1F0 1B0 1F1 1B1 1F2 1B2 1F3 1B3"],
    (2, 4, 4, 2, 0): ["0F0 0F1 2F0 2F1 2B0 0F2 2B1 0F3 0B0 2F2 0B1 2F3 2B2 2B3 0B2 0B3",
                      "1F0 1F1 3F0 3B0 3F1 3B1 1F2 1B0 1F3 1B1 3F2 3B2 3F3 3B3 1B2 1B3"],
    (2, 4, 4, 4, 1): ["0F0 0F1 0F2 0F3 2F0 2F1 2F2 2B0 2F3 2B1 2B2 2B3 0B0 0B1 0B2 0B3",
                      "1F0 1F1 1F2 1F3 3F0 3B0 3F1 3B1 3F2 3B2 3F3 3B3 1B0 1B1 1B2 1B3"],
    (4, 8, 4, 8, 0): [
        "0F0 0F1 0F2 0F3 0B0 0F4 0B1 0F5 0B2 0F6 0B3 0F7 0B4 0B5 0B6 0B7",
        "1F0 1F1 1F2 1B0 1F3 1B1 1F4 1B2 1F5 1B3 1F6 1B4 1F7 1B5 1B6 1B7",
        "2F0 2F1 2B0 2F2 2B1 2F3 2B2 2F4 2B3 2F5 2B4 2F6 2B5 2F7 2B6 2B7",
        "3F0 3B0 3F1 3B1 3F2 3B2 3F3 3B3 3F4 3B4 3F5 3B5 3F6 3B6 3F7 3B7"],
}


@pytest.mark.parametrize("key", list(GOLDEN))
def test_schedule_family_golden(key):
    p = S.PipeSchedParams(*key)
    assert fmt(p) == GOLDEN[key]
    S.validate_works(p)


def test_candidate_sets_and_step_expansion():
    pairs = lambda D, B, N: [(s.loop_batch, s.prefetch_fwd) for s in S.PipeSchedSet(D, B, N).scheds]
    assert pairs(4, 8, 8) == [(4, 0), (4, 1), (4, 2), (4, 3), (8, 0), (8, 1), (8, 2), (8, 3)]
    assert pairs(4, 8, 4) == [(8, 0), (8, 1), (8, 2), (8, 3)]
    steps = S.BeamScheduler(S.PipeSchedParams(2, 2, 2, 2, 0)).steps[0]
    assert " ".join(map(str, steps)) == (
        "RECV_ACT:0:0 FORWARD:0:0 SEND_ACT:0:0 RECV_ACT:0:1 FORWARD:0:1 SEND_ACT:0:1 "
        "RECV_GRAD:0:0 BACKWARD:0:0 SEND_GRAD:0:0 RECV_GRAD:0:1 BACKWARD:0:1 SEND_GRAD:0:1 "
        "OPTIMIZER_STEP:-1:-1")


@pytest.mark.parametrize("name", ["single_comm", "beam", "bfs", "dfs", "pipeless", "noskew"])
@pytest.mark.parametrize("D,B,N", [(2, 4, 2), (2, 4, 4), (3, 6, 6), (4, 8, 4)])
def test_every_scheduler_is_valid_and_deadlock_free(name, D, B, N):
    params = S.PipeSchedParams(D, B, N, min(B, D) if N > D else B, 0)
    sched = S.get_scheduler_class(name)(params)
    S.validate_works(params, sched.works)
    assert all(s[-1].work == S.StepWork.OPTIMIZER_STEP for s in sched.steps if s)
    assert all(st.work in (S.StepWork.RECV_ACT, S.StepWork.FORWARD, S.StepWork.SEND_ACT)
               for st in sched.get_eval_steps(0))
    nodes = [PipeNode(i, i % D, i, i + 1, comp_time=1.0, back_time=2.0) for i in range(N)]
    edges = [PipeEdge(i, i + 1, 1e6, 0.1) for i in range(N - 1)]
    pg = PipeGraph(nodes, edges, D)
    proxy = S.PipeSchedParams(D, B, N, params.loop_batch, 0)
    proxy.rank_works = sched.works
    assert pg.simulate(proxy).makespan > 0       # raises on a dependency deadlock


def test_mesh_arithmetic_table():
    assert parse_dp_mesh("-2,4") == (-2, 4) and parse_dp_mesh(None) is None
    a = MeshLayout.build(8, "-2,4")
    assert (a.pp_size, a.dp_size) == (4, 2)
    assert a.pp_group_ranks(5) == [4, 5, 6, 7] and a.dp_group_ranks(5) == [1, 5]
    assert [r for r in range(8) if a.is_main_rank(r)] == [3, 7]
    b = MeshLayout.build(8, "2,-4")
    assert (b.pp_size, b.dp_size) == (2, 4)
    assert b.pp_group_ranks(5) == [1, 5] and b.dp_group_ranks(5) == [4, 5, 6, 7]
    assert [r for r in range(8) if b.is_main_rank(r)] == [4, 5, 6, 7]
    c = MeshLayout.build(8, "-4,2")
    assert c.all_pp_groups() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    d = MeshLayout.build(4, None)
    assert d.pp_size == 4 and d.dp_size == 1 and d.is_main_rank(3) and not d.is_main_rank(0)
    assert check_main_rank(7, 8, "-2,4") and not check_main_rank(6, 8, "-2,4")
    with pytest.raises(ValueError):
        parse_dp_mesh("2,4")


def _random_graph(rng, n_stage, D):
    nodes = [PipeNode(i, i % D, i, i + 1, comp_time=rng.uniform(0.5, 3), back_time=rng.uniform(1, 6),
                      optim_time=rng.uniform(0, 1), act_mem=rng.uniform(1, 5), temp_mem=6,
                      weight=10) for i in range(n_stage)]
    edges = [PipeEdge(i, i + 1, 1e6, rng.uniform(0, 0.5)) for i in range(n_stage - 1)]
    for _ in range(n_stage // 2 if n_stage >= 3 else 0):       # skip connections
        a = rng.randrange(0, n_stage - 2)
        b = rng.randrange(a + 2, n_stage)
        if not any(e.start == a and e.end == b for e in edges):
            edges.append(PipeEdge(a, b, 1e6, rng.uniform(0, 0.5)))
    return PipeGraph(nodes, edges, D)


def test_cpp_evaluator_matches_python_oracle():
    from pfeife_b200.ops import _lib
    if _lib.host_lib() is None:
        pytest.skip("host library not built")
    rng = random.Random(0)
    for D, B, N in [(2, 4, 4), (3, 6, 6), (4, 8, 8), (4, 8, 4), (2, 3, 2)]:
        for sched in S.PipeSchedSet(D, B, N).scheds:
            pg = _random_graph(rng, N, D)
            assert pg.get_value(sched) == pytest.approx(pg.simulate(sched).makespan, rel=1e-12)


def test_peak_memory_walk():
    nodes = [PipeNode(0, 0, 0, 1, weight=100, act_mem=10, temp_mem=15, comp_time=1, back_time=2),
             PipeNode(1, 1, 1, 2, weight=50, act_mem=20, temp_mem=20, comp_time=1, back_time=2)]
    pg = PipeGraph(nodes, [PipeEdge(0, 1, 1, 0.1)], 2)
    sched = S.PipeSchedParams(2, 4, 2, 4, 0)        # rank 0 holds 2 activations at most
    assert pg.get_peak_memory(sched) == [100 + 10 + 15, 50 + 20]
    assert pg.fits(sched, [200, 200]) and not pg.fits(sched, [130, 200])


class _FakeCG:
    """A CompGraph stand-in with unit segments for planner tests."""

    def __init__(self, times, edge_bytes=1000, fb=2.0):
        from pfeife_b200.graph.comp_graph import CompEdge, CompNode
        self.nodes = [CompNode(i, [f"n{i}"], comp_time=t, act_mem=100, temp_mem=120,
                               weight=400, param_bytes=100) for i, t in enumerate(times)]
        self.edges = [CompEdge(i, i + 1, f"n{i}", edge_bytes) for i in range(len(times) - 1)]
        self.fb_ratio = fb

    def stage_bounds(self, pts):
        p = [0] + list(pts) + [len(self.nodes)]
        return [(p[i], p[i + 1]) for i in range(len(p) - 1)]

    def cross_edges(self, bounds):
        stage_of = {}
        for s, (lo, hi) in enumerate(bounds):
            for i in range(lo, hi):
                stage_of[i] = s
        out = {}
        for e in self.edges:
            a, b = stage_of[e.start], stage_of[e.end]
            if a != b:
                out[(a, b)] = out.get((a, b), 0) + e.weight
        return out


def test_beam_search_finds_brute_force_optimum_on_small_graphs():
    rng = random.Random(1)
    times = [rng.uniform(0.5, 4.0) for _ in range(12)]
    cg = _FakeCG(times)
    opt = PipeOption(device_cnt=3, batch_cnt=6, loop_cnt=1, prefetch_fwd=0, verbosity="error")
    gen = BeamSingleGenerator(cg, nvswitch_default(3), opt)
    plan = gen.gen_graph(6, None, None)
    sched = plan.sched
    best = min(gen._valuate_points(list(p), sched, None)[0]
               for p in itertools.combinations(range(1, 12), 2))
    assert plan.time <= best * 1.02
    assert plan.dep_graph is not None and plan.dep_graph.max_time == pytest.approx(plan.time)
    # the per-channel transfer order covers every inter-rank transfer exactly once
    n_comm = sum(len(v) for v in plan.dep_graph.channel_comms.values())
    assert n_comm == 2 * 2 * 6


def test_manual_split_points_and_every_partitioner():
    cg = _FakeCG([1.0] * 10)
    for name in ("beam_single", "beam_2", "random_walk", "same_mem", "same_time"):
        opt = PipeOption(device_cnt=2, batch_cnt=4, partitioner=name, loop_cnt=1, bench_seed=0,
                         verbosity="error")
        plan = get_pipe_class(name)(cg, None, opt).gen_graph(4, None, None)
        assert len(plan.split_points) == 1 and 1 <= plan.split_points[0] <= 9
    opt = PipeOption(device_cnt=2, batch_cnt=4, verbosity="error")
    plan = BeamSingleGenerator(cg, None, opt).gen_graph(4, None, [3])
    assert plan.split_points == [3] and len(plan.pipe_graph.nodes) == 2
    with pytest.raises(ValueError):
        BeamSingleGenerator(cg, None, opt).gen_graph(4, None, [0])


def test_link_model_fit_and_file_roundtrip(tmp_path):
    xs = [0.04, 0.16, 0.64, 2.5, 10, 39, 78, 156]
    ys = [0.02 if x <= 0.5 else 0.02 + 0.0014 * (x - 0.5) for x in xs]
    c, m, xb = fit_link(xs, ys)
    assert c == pytest.approx(0.02, abs=5e-3) and m == pytest.approx(0.0014, rel=0.1)
    b = DeviceBench()
    b.set_uniform(4, (c, m, xb))
    path = str(tmp_path / "dev.bench")
    b.save(path)
    b2 = DeviceBench()
    assert b2.load(path) and b2.params == b.params
    assert b2.send_time_rank(3, 1, 64 * 1024 ** 2) == b2.send_time_rank(1, 3, 64 * 1024 ** 2) > c
    assert b2.send_time_rank(2, 2, 1e9) == 0.0


def test_mesh_choice_prefers_dp_for_a_model_that_fits_and_pp_when_it_does_not():
    cg = _FakeCG([1.0] * 16)
    for n in cg.nodes:
        n.param_bytes, n.weight, n.act_mem, n.temp_mem = 1e6, 4e6, 1e6, 1.2e6
    opt = PipeOption(device_cnt=1, batch_size=4, batch_cnt=8, verbosity="error")
    bench = nvswitch_default(8)
    big = choose_mesh(cg, 8, opt, bench, device_mem=1e12)
    assert (big.pp, big.dp) == (1, 8) and big.dp_mesh == "-8,1"
    small = choose_mesh(cg, 8, opt, bench, device_mem=60e6)   # 64 MB of weights do not fit
    assert small.pp > 1 and small.pp * small.dp == 8
    assert dp_exposed_time(4e9, 1, bench) == 0.0 and dp_exposed_time(4e9, 8, bench) > 0


def test_plan_mesh_profiles_a_model_and_ranks_every_factorisation():
    """`plan_mesh` captures, profiles (CPU pass here) and returns one row per PP x DP = world."""
    import torch
    from pfeife_b200 import PipeOption, plan_mesh
    from pfeife_b200.models.vit import ViT, vit_config
    torch.manual_seed(0)
    model = ViT(vit_config("vit_tiny", num_layers=4, image_size=32, patch_size=8))
    opt = PipeOption(device_cnt=1, batch_size=4, batch_cnt=4, cpu_test=True)
    choice = plan_mesh(model, (torch.randn(4, 3, 32, 32),), opt, 4, torch.device("cpu"))
    assert sorted((pp, dp) for pp, dp, *_ in choice.table) == [(1, 4), (2, 2), (4, 1)]
    assert choice.pp * choice.dp == 4
    best = max(choice.table, key=lambda r: (r[4], r[3]))
    assert (choice.pp, choice.dp) == (best[0], best[1])
    assert choice.dp_mesh == (f"-{choice.dp},{choice.pp}" if choice.dp > 1 else f"{choice.pp}")


def test_schedule_picture_places_every_item_without_overlap(tmp_path):
    """The chart's boxes are the schedule's items at their simulated start times: every item
    appears once, boxes of one rank do not overlap, a backward never starts before its forward
    has ended, and the SVG and text forms carry all of them."""
    from pfeife_b200.parallel.gantt import save_schedule_svg, schedule_rows, schedule_table
    rng = random.Random(5)
    pg = _random_graph(rng, 4, 2)
    sched = S.PipeSchedParams(2, 4, 4, 2, 0)
    rows = schedule_rows(pg, sched)
    assert len(rows) == 4 * 4 * 2
    assert len({(x.stage, x.batch, x.is_fwd) for x in rows}) == len(rows)
    sim = pg.simulate(sched, record=True)
    for r in range(2):
        lane = [x for x in rows if x.rank == r]
        for a, b in zip(lane, lane[1:]):
            assert a.start + a.dur <= b.start + 1e-9
    when = {(x.stage, x.batch, x.is_fwd): x for x in rows}
    for (s, b, f), x in when.items():
        if not f:
            fw = when[(s, b, True)]
            assert fw.start + fw.dur <= x.start + 1e-9
    # (the makespan also holds the optimizer step that follows a rank's last backward)
    assert max(x.start + x.dur for x in rows) <= sim.makespan + 1e-9
    path = save_schedule_svg(pg, sched, str(tmp_path / "sched.svg"))
    svg = open(path).read()
    assert svg.startswith("<svg") and svg.count("<title>") == len(rows)
    assert len(schedule_table(pg, sched).splitlines()) == len(rows) + 1


@pytest.mark.parametrize("name", ["single_comm", "beam", "bfs", "dfs", "pipeless", "noskew"])
@pytest.mark.parametrize("D,B,N", [(2, 4, 2), (2, 4, 4), (3, 6, 6), (4, 8, 4), (4, 8, 8)])
def test_step_programs_keep_the_orderings_their_buffers_rely_on(name, D, B, N):
    """Every scheduler's per-rank programs, replayed on the host: receives precede their
    consumers, sends follow their producers, two micro-batches share a graph slot only when the
    first one's backward precedes the second one's forward, and all ranks together terminate
    under the transports' semantics (also with a skip connection across ranks)."""
    from pfeife_b200.runtime.hazards import program_hazards, replay_job
    from pfeife_b200.runtime.worker import inflight_slots
    params = S.PipeSchedParams(D, B, N, min(B, D) if N > D else B, 0)
    sched = S.get_scheduler_class(name)(params)
    stage_rank = {s: s % D for s in range(N)}
    for r in range(D):
        steps = sched.steps[r]
        slots, n_slots = inflight_slots(steps)
        assert program_hazards(steps, slots) == []
        assert n_slots <= B
    edges = [(i, i + 1) for i in range(N - 1)]
    assert replay_job(sched.steps, stage_rank, edges) == []
    if N >= 3:
        assert replay_job(sched.steps, stage_rank, edges + [(0, N - 1)]) == []


def test_hazard_checker_reports_broken_programs():
    from pfeife_b200.runtime.hazards import program_hazards, replay_job
    St, W = S.Step, S.StepWork
    ok = [St(W.RECV_ACT, 1, 0), St(W.FORWARD, 1, 0), St(W.RECV_ACT, 1, 1), St(W.FORWARD, 1, 1),
          St(W.BACKWARD, 1, 0), St(W.SEND_GRAD, 1, 0), St(W.BACKWARD, 1, 1), St(W.SEND_GRAD, 1, 1),
          St(W.OPTIMIZER_STEP, -1, -1)]
    assert program_hazards(ok, {(1, 0): 0, (1, 1): 1}) == []
    # both micro-batches in one slot while both are in flight
    assert any("slot" in p for p in program_hazards(ok, {(1, 0): 0, (1, 1): 0}))
    # a forward ahead of its receive, a send ahead of its backward
    bad = [ok[1], ok[0]] + ok[2:4] + [ok[5], ok[4]] + ok[6:]
    msgs = program_hazards(bad, {(1, 0): 0, (1, 1): 1})
    assert any("inputs are not there" in p for p in msgs) and any("nothing to send" in p for p in msgs)
    # two ranks that each wait for the other's message first
    r0 = [St(W.RECV_GRAD, 0, 0), St(W.FORWARD, 0, 0), St(W.SEND_ACT, 0, 0)]
    r1 = [St(W.RECV_ACT, 1, 0), St(W.FORWARD, 1, 0), St(W.BACKWARD, 1, 0), St(W.SEND_GRAD, 1, 0)]
    assert any("waits for ever" in p for p in replay_job([r0, r1], {0: 0, 1: 1}, [(0, 1)]))
