"""mp_launch.py: rank environment of the three launchers and an end-to-end torchrun launch."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mod():
    spec = importlib.util.spec_from_file_location("mp_launch", os.path.join(ROOT, "mp_launch.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_python_launcher_ranks_and_child_command():
    m = _mod()
    args = m.parse_args(["--world_size", "8", "--nnodes", "2", "--node_rank", "1",
                         "--dp_mesh=-2,4", "--cpu", "train.py", "--batch_size", "4"])
    env = m.get_python_env(args, 3)
    assert (env["RANK"], env["LOCAL_RANK"], env["WORLD_SIZE"], env["DP_MESH"]) == \
        ("7", "3", "8", "-2,4")
    assert env["PFEIFE_CPU"] == "1" and env["MASTER_ADDR"] == "127.0.0.1"
    argv = m.child_argv(args)
    assert "--run_proc" in argv and "--dp_mesh=-2,4" in argv
    assert argv[argv.index("--launcher") + 1] == "python"
    assert argv[argv.index("--") + 1:] == ["train.py", "--batch_size", "4"]


def test_slurm_tasks_take_their_rank_from_slurm():
    m = _mod()
    args = m.parse_args(["--launcher", "slurm", "--world_size", "16", "--nnodes", "2", "x.py"])
    env = m.get_slurm_env(args, {"SLURM_PROCID": "11", "SLURM_LOCALID": "3", "SLURM_NTASKS": "16",
                                 "SLURM_NNODES": "2", "SLURM_NODEID": "1"})
    assert (env["RANK"], env["LOCAL_RANK"], env["WORLD_SIZE"], env["NNODES"], env["NODE_RANK"]) \
        == ("11", "3", "16", "2", "1")
    assert m.child_argv(args)[m.child_argv(args).index("--launcher") + 1] == "slurm"


def test_torchrun_launcher_trains_a_two_rank_pipeline(tmp_path):
    out = str(tmp_path / "r.json")
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--launcher", "torchrun", "--cpu",
           "--world_size", "2", "--master_port", "29688",
           os.path.join(ROOT, "tests", "scripts", "train_check.py"), "--cpu",
           "--no_bench_optimizer", "--ctrl_timeout", "120", "--out", out, "--model", "mlp",
           "--device_cnt", "2", "--batch_size", "4", "--batch_cnt", "2", "--steps", "2"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=420, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-4000:]
    with open(out) as f:
        res = json.load(f)
    assert res["param_diff"] <= 1e-5
