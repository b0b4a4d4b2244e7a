"""Two-GPU runs (one process per GPU, NCCL + peer memory) through ``mp_launch.py``."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_port = [29811]


def launch(tmp_path, world, script_args, dp_mesh=None, tag="r", timeout=420):
    out = str(tmp_path / f"{tag}.json")
    _port[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--world_size", str(world),
           "--master_port", str(_port[0])]
    if dp_mesh:
        cmd.append(f"--dp_mesh={dp_mesh}")
    cmd += [os.path.join(ROOT, "tests", "scripts", "train_check.py"), "--no_bench_optimizer",
            "--ctrl_timeout", "120", "--out", out] + script_args
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=timeout, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-4000:]
    with open(out) as f:
        return json.load(f), out


@pytest.mark.parametrize("extra", [[], ["--cuda_graphs"], ["--cuda_graphs", "--loop_cnt", "2"]],
                         ids=["eager", "graphs", "graphs_looped"])
def test_pp2_gpu_matches_single_process(tmp_path, extra):
    """Two pipeline ranks against the un-pipelined loop: eagerly, with every (stage, slot)
    replayed from CUDA graphs (the gradients a replayed stage hands upstream come from its
    static inputs), and with two stages per rank, where stages both receive and send."""
    res, _ = launch(tmp_path, 2, ["--model", "vit_small", "--device_cnt", "2", "--batch_size", "4",
                                  "--batch_cnt", "4", "--steps", "4", "--optimizer", "adamw",
                                  "--lr", "0.001", "--mixed_precision", "bf16"] + extra)
    for a, b in zip(res["losses"], res["ref_losses"]):
        assert a == pytest.approx(b, rel=5e-2, abs=5e-2)
    assert res["param_diff"] < 2e-2
    if extra:
        assert res["graphs"] > 0 and res["graphs_failed"] == 0, res


def test_fused_dp_equals_nccl_dp(tmp_path):
    common = ["--model", "vit_small", "--device_cnt", "1", "--batch_size", "4", "--batch_cnt", "2",
              "--steps", "4", "--optimizer", "adamw", "--lr", "0.001", "--mixed_precision", "bf16"]
    fused, out_f = launch(tmp_path, 2, common, dp_mesh="-2,1", tag="fused")
    nccl, out_n = launch(tmp_path, 2, common + ["--no_fused_dp"], dp_mesh="-2,1", tag="nccl")
    with open(out_f + ".dp0") as f:
        fused_other = json.load(f)
    # replicas hold identical weights, and the fused path lands where the NCCL baseline does
    assert fused["param_checksum"] == pytest.approx(fused_other["param_checksum"], rel=1e-7)
    assert fused["param_checksum"] == pytest.approx(nccl["param_checksum"], rel=1e-4, abs=1e-3)
    for a, b in zip(fused["losses"], nccl["losses"]):
        assert a == pytest.approx(b, rel=2e-2, abs=2e-2)


def test_fused_dp_on_four_replicas_equals_nccl_dp(tmp_path):
    """The four-rank instantiation of the fused step (two vectors per peer in flight)."""
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 CUDA devices")
    common = ["--model", "vit_small", "--device_cnt", "1", "--batch_size", "4", "--batch_cnt", "2",
              "--steps", "4", "--optimizer", "adamw", "--lr", "0.001", "--mixed_precision", "bf16"]
    fused, out_f = launch(tmp_path, 4, common, dp_mesh="-4,1", tag="fused4")
    nccl, _ = launch(tmp_path, 4, common + ["--no_fused_dp"], dp_mesh="-4,1", tag="nccl4")
    for r in (0, 1, 2):          # the main process is the last replica
        with open(out_f + f".dp{r}") as f:
            other = json.load(f)
        assert fused["param_checksum"] == pytest.approx(other["param_checksum"], rel=1e-7)
    assert fused["param_checksum"] == pytest.approx(nccl["param_checksum"], rel=1e-4, abs=1e-3)
    for a, b in zip(fused["losses"], nccl["losses"]):
        assert a == pytest.approx(b, rel=2e-2, abs=2e-2)


@pytest.mark.parametrize("graphs", [False, True])
def test_row_sharded_weights_match_replicated_weights(tmp_path, graphs):
    """--use_fsdp with the fused data-parallel step: after the optimizer step every weight matrix
    is current only in the rows its rank owns and the first GEMM that reads it gathers the rest.
    Training must land where the fully replicated run lands, eagerly and under CUDA graphs."""
    common = ["--model", "vit_wide", "--device_cnt", "1", "--batch_size", "4", "--batch_cnt", "2",
              "--steps", "5", "--optimizer", "adamw", "--lr", "0.001", "--mixed_precision", "bf16"]
    if graphs:
        common.append("--cuda_graphs")
    sharded, out_s = launch(tmp_path, 2, common + ["--use_fsdp"], dp_mesh="-2,1", tag="sharded")
    repl, _ = launch(tmp_path, 2, common, dp_mesh="-2,1", tag="repl")
    with open(out_s + ".dp0") as f:
        other = json.load(f)
    assert sharded["param_checksum"] == pytest.approx(other["param_checksum"], rel=1e-7)
    assert sharded["param_checksum"] == pytest.approx(repl["param_checksum"], rel=1e-6, abs=1e-4)
    for a, b in zip(sharded["losses"], repl["losses"]):
        assert a == pytest.approx(b, rel=1e-3, abs=1e-3)


def _overflow_run(tmp_path, world, mesh, device_cnt):
    res, out = launch(tmp_path, world, ["--model", "vit_small", "--device_cnt", str(device_cnt),
                                        "--batch_size", "4", "--batch_cnt", "2", "--steps", "3",
                                        "--optimizer", "adamw", "--lr", "0.001",
                                        "--mixed_precision", "fp16", "--two_groups",
                                        "--inject_inf", "1"], dp_mesh=mesh, tag="ovf")
    with open(out + ".dp0") as f:
        other = json.load(f)
    for r in (res, other):
        # the overflowing step was skipped by every parameter of both groups on every rank
        assert r["opt_steps"] == [2], r["opt_steps"]
        assert r["loss_scale"] == 32768.0
    assert res["param_checksum"] == pytest.approx(other["param_checksum"], rel=1e-7)


def test_overflow_on_one_replica_skips_both_groups_on_both_replicas(tmp_path):
    """fp16, two optimizer groups, fused data parallelism: one replica's gradients overflow in
    step 1.  Both replicas skip that step for BOTH groups, halve the scale once and keep
    identical weights; Adam's step count leaves the skipped step out."""
    _overflow_run(tmp_path, 2, "-2,1", 1)


def test_overflow_is_agreed_over_pipeline_and_replicas(tmp_path):
    """The same with two pipeline stages per replica (PP2 x DP2): the stage that did not
    overflow itself skips too, and every rank keeps the same scale."""
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 CUDA devices")
    _overflow_run(tmp_path, 4, "-2,2", 2)


def test_checkpoint_resume_under_fused_dp(tmp_path):
    """The fused data-parallel step keeps Adam moments only on the rank that owns each shard;
    a checkpoint assembles them and a restore hands every rank its shard back: the two steps
    after the checkpoint repeat exactly after the restore, on both replicas."""
    res, out = launch(tmp_path, 2, ["--model", "vit_small", "--device_cnt", "1", "--batch_size",
                                    "4", "--batch_cnt", "2", "--steps", "2", "--optimizer",
                                    "adamw", "--lr", "0.001", "--mixed_precision", "bf16",
                                    "--resume_check"], dp_mesh="-2,1", tag="resume")
    with open(out + ".dp0") as f:
        other = json.load(f)
    for r in (res, other):
        for a, b in zip(r["resume_first"], r["resume_second"]):
            assert a == pytest.approx(b, abs=1e-5, rel=1e-5)
        assert r["resume_first"][0] != pytest.approx(r["resume_first"][1], abs=1e-9)


def test_allgather_fused_into_gemm(tmp_path):
    out = str(tmp_path / "ag.json")
    _port[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--world_size", "2", "--all_main",
           "--master_port", str(_port[0]),
           os.path.join(ROOT, "tests", "scripts", "allgather_gemm_check.py"), "--out", out,
           "--M", "1000", "--N", "1024", "--K", "320", "--iters", "3"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:]
    with open(out) as f:
        res = json.load(f)
    assert res["gathered_ok"] and res["err"] < 0.15


def test_thread_runtime_on_two_gpus_matches_the_plain_loop():
    """The single-process runtime (one thread per device, activations moved by peer copies on
    side streams) through ``benchmark_local.py --check_valid`` on two GPUs: pipelined training
    tracks the un-pipelined loop step by step."""
    import re
    cmd = [sys.executable, os.path.join(ROOT, "benchmark_local.py"), "--model", "vit_tiny",
           "--device_cnt", "2", "--batch_size", "2", "--batch_cnt", "4", "--check_valid",
           "--valid_steps", "3"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=420, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-4000:]
    d = [float(x) for x in re.findall(r"diff percentage: (-?[0-9.]+)%", r.stdout)]
    assert len(d) == 3 and max(abs(x) for x in d) < 1.0, r.stdout[-2000:]
