"""The example trainers run end to end on CPU ranks (gloo) at reduced shapes: two pipeline
stages, checkpoints written and resumed, the throughput line printed."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PORT = [25310]


def _launch(script, extra, world=2, mesh=None, timeout=600):
    _PORT[0] += 1
    cmd = [sys.executable, os.path.join(ROOT, "mp_launch.py"), "--world_size", str(world), "--cpu",
           "--master_port", str(_PORT[0])]
    if mesh:
        cmd.append(f"--dp_mesh={mesh}")
    cmd += [os.path.join(ROOT, "examples", script)] + extra
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    m = re.search(r"^throughput: +([0-9.]+) it/s, +([0-9.]+) samples/s, final loss ([-0-9.naninf]+)",
                  p.stdout, re.M)
    assert m, p.stdout[-2000:]
    return float(m.group(1)), float(m.group(3)), p.stdout


COMMON = ["--batch_cnt", "2", "--warmup_iters", "1", "--log_every", "1", "--dataset_len", "32"]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("precision", [None, "fp16"])
def test_vit_trainer_checkpoints_and_resumes(tmp_path, precision):
    """Under fp16 the first steps overflow at the initial loss scale and are skipped: the
    checkpoint has to carry the scale the job backed off to and the optimizer's own step count
    (which leaves the skipped steps out), or the resumed run diverges from the straight one."""
    base = ["--model", "vit_tiny", "--image_size", "32", "--num_layers", "4", "--batch_size", "2"] + COMMON
    if precision:
        base += ["--mixed_precision", precision]
    out = str(tmp_path / "ck")
    its, loss_a, log = _launch("train_vit.py", base + ["--iter_cnt", "4", "--output_dir", out,
                                                       "--checkpointing_steps", "2"])
    assert its > 0 and loss_a == loss_a
    assert sorted(os.listdir(out)) == ["checkpoint-2.pt", "checkpoint-4.pt"]
    ck = torch.load(os.path.join(out, "checkpoint-2.pt"), map_location="cpu", weights_only=False)
    assert ck["step"] == 2 and "pos_embed" in "".join(ck["model"].keys())
    # AdamW moments come back under the parameter names
    name = next(k for k in ck["optimizer"] if not k.startswith("__"))
    assert name in ck["model"] and {"exp_avg", "exp_avg_sq"} <= set(ck["optimizer"][name])
    assert ("__loss_scaler__" in ck["optimizer"]) == bool(precision)
    # steps 3 and 4 again from the checkpoint of step 2: same data order, same state, same loss
    _, loss_b, _ = _launch("train_vit.py", base + ["--iter_cnt", "4", "--resume_from",
                                                   os.path.join(out, "checkpoint-2.pt")])
    assert loss_b == pytest.approx(loss_a, rel=1e-4 if not precision else 5e-3, abs=1e-5)


@pytest.mark.timeout(900)
def test_llama_trainer_tied_embeddings_two_groups():
    its, loss, log = _launch("train_llama.py", ["--model", "llama_tiny", "--block_size", "16",
                                               "--per_device_train_batch_size", "2", "--iter_cnt", "4",
                                               "--tie_embeddings", "--num_warmup_steps", "2",
                                               "--weight_decay", "0.1", "--learning_rate", "1e-3"]
                             + COMMON)
    assert its > 0 and 4.0 < loss < 6.5      # ln(256) = 5.55 at the start
    assert log.count("throughput ") == 3


@pytest.mark.timeout(900)
def test_llama_trainer_data_parallel_from_a_file(tmp_path):
    ids = torch.randint(0, 256, (16, 16))
    path = str(tmp_path / "ids.pt")
    torch.save((ids,), path)
    its, loss, _ = _launch("train_llama.py", ["--model", "llama_tiny", "--block_size", "16",
                                             "--per_device_train_batch_size", "2", "--iter_cnt", "3",
                                             "--data_file", path] + COMMON, mesh="-2,1")
    assert its > 0 and 4.0 < loss < 6.5


@pytest.mark.timeout(1200)
def test_sdxl_trainer_min_snr_v_prediction():
    its, loss, _ = _launch("train_sdxl.py", ["--model", "unet_tiny", "--resolution", "64",
                                            "--train_batch_size", "2", "--iter_cnt", "3",
                                            "--snr_gamma", "5", "--prediction_type", "v_prediction",
                                            "--noise_offset", "0.05", "--proportion_empty_prompts",
                                            "0.5"] + COMMON, timeout=1100)
    assert its > 0 and 0.0 < loss < 10.0
