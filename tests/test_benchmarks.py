"""The benchmark drivers on CPU: validity check (pipelined against un-pipelined, tied weights,
foreign models), the timing line, and a first step that fails must end the job, not stall it."""
import os
import re
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PORT = [25510]


def _mp(extra, world=2, timeout=600):
    _PORT[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--world_size", str(world), "--cpu",
           "--master_port", str(_PORT[0]), os.path.join(ROOT, "benchmark_mp.py")] + extra
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def _local(extra, timeout=600):
    cmd = [sys.executable, os.path.join(ROOT, "benchmark_local.py"), "--cpu"] + extra
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def _diffs(out):
    return [float(x) for x in re.findall(r"diff percentage: (-?[0-9.]+)%", out)]


SMALL = ["--batch_size", "2", "--batch_cnt", "2"]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model", ["toy", "llama_tiny", "unet_tiny"])
def test_mp_check_valid(model):
    p = _mp(["--model", model, "--check_valid", "--valid_steps", "3"] + SMALL)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    d = _diffs(p.stdout)
    assert len(d) == 3 and max(abs(x) for x in d) < 0.5


@pytest.mark.timeout(900)
def test_mp_timing_line():
    p = _mp(["--model", "vit_tiny", "--repeat", "2"] + SMALL)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert re.search(r"mean latency [0-9.e-]+ / std.dev. [0-9.e-]+ across 2 runs", p.stdout)


@pytest.mark.timeout(900)
def test_local_check_valid_and_records():
    p = _local(["--model", "toy", "--device_cnt", "2", "--check_valid", "--valid_steps", "3"] + SMALL)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert len(_diffs(p.stdout)) == 3 and max(abs(x) for x in _diffs(p.stdout)) < 0.5
    p = _local(["--model", "vit_tiny", "--device_cnt", "2", "--repeat", "2"] + SMALL)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert "mean latency" in p.stdout and re.search(r"stage 0: forward [0-9.]+ ms", p.stdout)


@pytest.mark.timeout(300)
def test_a_failed_first_step_ends_the_job():
    """Three compute nodes cannot fill four stages: the main rank raises before it has a plan,
    and the three ranks waiting for that plan must be released."""
    t0 = time.time()
    p = _mp(["--model", "toy", "--repeat", "1"] + SMALL, world=4, timeout=240)
    assert p.returncode != 0
    assert "no captured graph is eligible for pipelining" in p.stderr + p.stdout
    assert time.time() - t0 < 200


def test_reference_arm_sweeps_the_reference_meshes_best_first():
    """The reference arm tries the reference's own PP x DP layouts for the world size (short
    pipelines replicated first, one pipeline over everything last) and names them like the
    native arm names its parallelism."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "reference_arm", os.path.join(root, "baseline", "reference_arm.py"))
    arm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(arm)
    assert arm._candidate_meshes(8) == ["-4,2", "-2,4", "8"]
    assert arm._candidate_meshes(4) == ["-2,2", "4"]
    assert arm._candidate_meshes(2) == ["2"]
    assert [arm._mesh_name(m) for m in arm._candidate_meshes(8)] == ["pp2xdp4", "pp4xdp2", "pp8"]
