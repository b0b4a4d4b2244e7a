"""Multi-process runs on CPU (gloo) through ``mp_launch.py`` and the public API: losses and
final parameters must equal plain single-process training (asserted, not printed)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_port = [29611]


def launch(tmp_path, world, script_args, dp_mesh=None, timeout=420):
    out = str(tmp_path / "result.json")
    _port[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--cpu", "--world_size", str(world),
           "--master_port", str(_port[0])]
    if dp_mesh:
        cmd.append(f"--dp_mesh={dp_mesh}")
    cmd += [os.path.join(ROOT, "tests", "scripts", "train_check.py"), "--cpu",
            "--no_bench_optimizer", "--ctrl_timeout", "120", "--out", out] + script_args
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-4000:]
    with open(out) as f:
        return json.load(f), out


def assert_equal_training(res, tol=1e-5):
    assert len(res["losses"]) == len(res["ref_losses"]) > 0
    for a, b in zip(res["losses"], res["ref_losses"]):
        assert a == pytest.approx(b, abs=tol, rel=tol)
    assert res["param_diff"] <= tol


def test_vit_tiny_pp2_baseline_config(tmp_path):
    """ViT-Tiny/16 fp32, 12 layers, hidden 192, 224x224 images, 10 classes, SGD lr 0.01,
    batch_size 4, batch_cnt 4, world_size 2 on gloo."""
    res, _ = launch(tmp_path, 2, ["--model", "vit_tiny", "--device_cnt", "2", "--batch_size", "4",
                                  "--batch_cnt", "4", "--steps", "2", "--lr", "0.01"])
    assert_equal_training(res, tol=2e-4)
    assert res["state_dict_keys"] > 100


def test_tied_weights_across_ranks_adam(tmp_path):
    res, _ = launch(tmp_path, 2, ["--model", "tied", "--device_cnt", "2", "--batch_size", "2",
                                  "--batch_cnt", "4", "--steps", "3", "--optimizer", "adam",
                                  "--loop_cnt", "1"])
    assert_equal_training(res, tol=1e-5)


def test_skip_connections_looped_pp2(tmp_path):
    res, _ = launch(tmp_path, 2, ["--model", "skip", "--device_cnt", "2", "--batch_size", "2",
                                  "--batch_cnt", "4", "--steps", "3", "--loop_cnt", "2",
                                  "--check_eval"])
    assert_equal_training(res, tol=1e-5)
    assert res["eval_diff"] <= 1e-5


def test_pp3_manual_split_gpipe_scheduler(tmp_path):
    res, _ = launch(tmp_path, 3, ["--model", "mlp", "--device_cnt", "3", "--batch_size", "2",
                                  "--batch_cnt", "3", "--steps", "2", "--split_points", "8,16",
                                  "--scheduler", "bfs", "--optimizer", "adamw"])
    assert_equal_training(res, tol=1e-5)
    assert res["opt_state_keys"]


def test_dp2_x_pp2_replicas_stay_identical(tmp_path):
    res, out = launch(tmp_path, 4, ["--model", "mlp", "--device_cnt", "2", "--batch_size", "2",
                                    "--batch_cnt", "2", "--steps", "3"], dp_mesh="-2,2")
    with open(out + ".dp0") as f:
        other = json.load(f)
    assert res["param_checksum"] == pytest.approx(other["param_checksum"], rel=1e-9)
    assert res["losses"] != other["losses"]      # replicas saw different data


def test_replicas_install_one_plan_whatever_they_would_measure(tmp_path):
    """Two replicas whose own profiles would differ (every profiling rank gets different segment
    times) still install the same split points: only the first replica profiles and plans."""
    res, out = launch(tmp_path, 4, ["--model", "mlp", "--device_cnt", "2", "--batch_size", "2",
                                    "--batch_cnt", "2", "--steps", "2", "--skew_profile"],
                      dp_mesh="-2,2")
    with open(out + ".dp0") as f:
        other = json.load(f)
    assert res["split_points"] and res["split_points"] == other["split_points"]
    assert res["param_checksum"] == pytest.approx(other["param_checksum"], rel=1e-9)


def test_llama_tied_embeddings_looped(tmp_path):
    res, _ = launch(tmp_path, 2, ["--model", "llama_tiny", "--device_cnt", "2", "--batch_size", "2",
                                  "--batch_cnt", "4", "--steps", "2"])
    assert_equal_training(res, tol=1e-5)


def test_unet_long_skip_edges_and_many_inputs(tmp_path):
    res, _ = launch(tmp_path, 2, ["--model", "unet_tiny", "--device_cnt", "2", "--batch_size", "2",
                                  "--batch_cnt", "4", "--steps", "2"])
    assert_equal_training(res, tol=1e-5)


def test_checkpoint_resume_repeats_the_same_steps(tmp_path):
    """gather_params(with_optimizer=True) -> load_params restores parameters, Adam moments and
    the step count on every rank: the two steps after the checkpoint give the same losses when
    they are repeated after the restore."""
    res, _ = launch(tmp_path, 2, ["--model", "mlp", "--device_cnt", "2", "--batch_size", "4",
                                  "--batch_cnt", "2", "--steps", "2", "--optimizer", "adam",
                                  "--lr", "0.01", "--resume_check"])
    assert len(res["resume_first"]) == 2
    for a, b in zip(res["resume_first"], res["resume_second"]):
        assert a == pytest.approx(b, abs=1e-6, rel=1e-6)
    # and training did move between the two steps (the check is not vacuous)
    assert res["resume_first"][0] != pytest.approx(res["resume_first"][1], abs=1e-9)


@pytest.mark.parametrize("fail_rank", [0, 1])
def test_a_rank_that_raises_takes_the_job_down(tmp_path, fail_rank):
    """Failure detection on the host: one rank raises before its first step; the launcher notices
    the dead child, ends the others and reports a non-zero exit instead of hanging."""
    import time
    out = str(tmp_path / "result.json")
    _port[0] += 1
    # --all_main: every rank runs the script, so the failing rank can be a pipeline worker
    # (rank 0) as well as the pipeline's main rank (rank 1)
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--cpu", "--world_size", "2",
           "--all_main", "--master_port", str(_port[0]),
           os.path.join(ROOT, "tests", "scripts", "train_check.py"), "--cpu",
           "--no_bench_optimizer", "--ctrl_timeout", "30", "--out", out, "--model", "mlp",
           "--device_cnt", "2", "--batch_size", "4", "--batch_cnt", "2", "--steps", "2",
           "--fail_rank", str(fail_rank)]
    t0 = time.time()
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=240, cwd=ROOT)
    assert r.returncode != 0
    assert "injected host-side failure" in r.stdout
    assert time.time() - t0 < 200
    assert not os.path.exists(out)


def test_manager_front_end_owns_loss_and_optimizer(tmp_path):
    """``PipeManager(model, loss_fn, option).run(target, *inputs)`` over a 2-rank pipeline:
    training, eval and gather_params against a plain loop."""
    out = str(tmp_path / "mgr.json")
    _port[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--cpu", "--world_size", "2",
           "--master_port", str(_port[0]),
           os.path.join(ROOT, "tests", "scripts", "manager_check.py"), "--cpu",
           "--no_bench_optimizer", "--ctrl_timeout", "120", "--out", out, "--device_cnt", "2",
           "--batch_size", "4", "--batch_cnt", "2"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=420, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-4000:]
    with open(out) as f:
        res = json.load(f)
    assert_equal_training(res)
    assert res["eval_diff"] <= 1e-5
