"""Training-equality check driven through the public API (run by the tests under
``mp_launch.py``): trains a model for a few steps through the pipeline and through a plain
single-process loop with the same optimizer, and writes losses and the largest parameter
difference to ``--out`` as JSON (only the global main process writes)."""
import argparse
import copy
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, ops, partial_compiler  # noqa
from pfeife_b200.models.toy import DeepMLP, SkipNet, TiedMLP  # noqa
from pfeife_b200.models.vit import ViT, vit_config  # noqa
from pfeife_b200.utils import set_seed  # noqa


def _clf(model, make_x, n_cls):
    def batch(n, g):
        return (torch.randn(make_x(n).shape, generator=g), torch.randint(0, n_cls, (n,), generator=g))

    def loss(call, x, y):
        # the fused loss kernel runs in the front-end threads on GPU ranks
        return ops.cross_entropy(call(x).float(), y)
    return model, batch, loss


def build(name):
    """-> (model, make_batch(n, generator) -> tensors, loss(callable_model, *tensors))."""
    if name == "mlp":
        return _clf(DeepMLP(16, 8, 10), (lambda n: torch.randn(n, 16)), 10)
    if name == "tied":
        return _clf(TiedMLP(10, 3), (lambda n: torch.randn(n, 10)), 10)
    if name == "skip":
        return _clf(SkipNet(16, 3), (lambda n: torch.randn(n, 16)), 16)
    if name == "vit_tiny":
        return _clf(ViT(vit_config("vit_tiny")), (lambda n: torch.randn(n, 3, 224, 224)), 10)
    if name == "vit_small":
        cfg = vit_config("vit_tiny", num_layers=4, image_size=32, patch_size=8)
        return _clf(ViT(cfg), (lambda n: torch.randn(n, 3, 32, 32)), 10)
    if name == "vit_wide":      # matrices large enough for the row-sharded (deferred gather) path
        cfg = vit_config("vit_tiny", num_layers=2, hidden_size=512, num_heads=8, mlp_dim=2048,
                         image_size=32, patch_size=8)
        return _clf(ViT(cfg), (lambda n: torch.randn(n, 3, 32, 32)), 10)
    if name == "llama_tiny":
        from pfeife_b200.models.llama import Llama, causal_lm_loss, llama_config
        model = Llama(llama_config("llama_tiny", tie_embeddings=True))
        return (model, lambda n, g: (torch.randint(0, 256, (n, 16), generator=g),),
                lambda call, ids: causal_lm_loss(call(ids).float(), ids))
    if name == "unet_tiny":
        from pfeife_b200.models.unet import UNet, unet_config
        model = UNet(unet_config("unet_tiny"))

        def batch(n, g):
            r = lambda *s: torch.randn(*s, generator=g)
            return (r(n, 4, 16, 16), torch.randint(0, 1000, (n,), generator=g), r(n, 7, 32),
                    r(n, 16), r(n, 6), r(n, 4, 16, 16))

        def loss(call, lat, t, txt, pooled, ids, noise):
            return F.mse_loss(call(lat, t, txt, pooled, ids).float(), noise)
        return model, batch, loss
    raise ValueError(name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mlp")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--out", required=True)
    ap.add_argument("--optimizer", default="sgd")
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--check_eval", action="store_true")
    ap.add_argument("--resume_check", action="store_true")
    ap.add_argument("--fail_rank", type=int, default=-1,
                    help="this global rank raises an exception on the host before its first step "
                         "(failure-detection test; no device work is in flight)")
    ap.add_argument("--inject_inf", type=int, default=-1,
                    help="at this step the first replica's inputs are infinite, so its "
                         "gradients overflow (dynamic loss scaling must skip the step everywhere)")
    ap.add_argument("--two_groups", action="store_true",
                    help="matrices and vectors in two optimizer groups")
    ap.add_argument("--skew_profile", action="store_true",
                    help="every rank that profiles gets segment times of its own (seeded by its "
                         "rank), as timing noise on real devices would give it")
    PipeOption.add_arguments(ap)
    args = ap.parse_args()

    state = initialize_pfeife()
    if args.fail_rank == state.rank:
        raise RuntimeError(f"injected host-side failure on rank {state.rank}")
    if not state.is_main_rank:
        # only under ``mp_launch.py --all_main`` (the launcher runs worker ranks itself otherwise)
        from pfeife_b200.runtime.partial import worker_loop
        worker_loop()
        return
    option = PipeOption.from_args(args)
    if args.skew_profile:
        import random

        from pfeife_b200.runtime import partial as _partial
        plain = _partial.gen_comp_graph_cpu

        def skewed(captured, call_args, opt):
            cg, out = plain(captured, call_args, opt)
            rng = random.Random(1234 + state.rank)
            for node in cg.nodes:
                node.comp_time = rng.uniform(0.2, 5.0)
            return cg, out
        _partial.gen_comp_graph_cpu = skewed
    set_seed(0)
    model, make_batch, loss_fn = build(args.model)
    ref = copy.deepcopy(model)
    dev = state.device
    model.to(dev)
    def param_sets(m):
        if not args.two_groups:
            return m.parameters()
        ps = list(m.parameters())
        return [{"params": [p for p in ps if p.dim() >= 2]},
                {"params": [p for p in ps if p.dim() < 2], "weight_decay": 0.0}]

    mk = lambda m: (torch.optim.SGD(param_sets(m), lr=args.lr) if args.optimizer == "sgd" else
                    torch.optim.AdamW(param_sets(m), lr=args.lr, weight_decay=0.01)
                    if args.optimizer == "adamw" else torch.optim.Adam(param_sets(m), lr=args.lr))
    opt, ropt = mk(model), mk(ref)
    sched = torch.optim.lr_scheduler.StepLR(opt, 1, gamma=0.5)
    rsched = torch.optim.lr_scheduler.StepLR(ropt, 1, gamma=0.5)

    runner = PartialRunner(option, opt)
    cm = torch.compile(model, backend=partial_compiler)

    def exec_fn(*batch):
        loss = loss_fn(cm, *batch)
        runner.scaler.scale(loss).backward()
        return loss.detach().cpu()

    runner.set_exec_fn(exec_fn)
    n = option.batch_size * option.batch_cnt
    g = torch.Generator().manual_seed(100 + state.dp_rank)
    losses, ref_losses = [], []
    for step in range(args.steps):
        batch = make_batch(n, g)
        if step == args.inject_inf and state.dp_rank == 0:
            batch = tuple(t * float("inf") if t.is_floating_point() else t for t in batch)
        out = runner.step(*[t.to(dev) for t in batch])
        losses.append([float(l) for l in out])
        sched.step()
        if state.dp_size == 1:
            ropt.zero_grad()
            cur = []
            for mb in zip(*[t.chunk(option.batch_cnt) for t in batch]):
                l = loss_fn(ref, *mb)
                l.backward()
                cur.append(float(l.detach()))
            ropt.step()
            rsched.step()
            ref_losses.append(cur)
    result = {"losses": losses, "ref_losses": ref_losses}
    if args.check_eval:
        x = make_batch(n, g)[0]
        runner.set_exec_fn(lambda x: cm(x).detach().cpu())
        got = runner.eval_step(x.to(dev))
        runner.gather_params()
        with torch.no_grad():
            want = model.cpu()(x)
        result["eval_diff"] = float((torch.cat(got) - want).abs().max())
        model.to(dev)
    if args.resume_check:
        # checkpoint, train two more steps, restore the checkpoint, repeat the same two steps:
        # parameters, optimizer moments and step count all have to come back
        saved_opt = runner.gather_params(with_optimizer=True)
        saved = {k: v.detach().clone() for k, v in model.state_dict().items()}
        g2 = torch.Generator().manual_seed(777 + state.dp_rank)
        batches = [make_batch(n, g2) for _ in range(2)]

        def two_steps():
            return [[float(l) for l in runner.step(*[t.to(dev) for t in b])] for b in batches]

        result["resume_first"] = two_steps()
        runner.load_params(saved, saved_opt)
        result["resume_second"] = two_steps()
    opt_state = runner.gather_params(with_optimizer=True)
    diff = 0.0
    if state.dp_size == 1:
        for (k, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            diff = max(diff, float((p.detach().cpu() - q.detach()).abs().max()))
    result["param_diff"] = diff
    result["opt_state_keys"] = sorted(opt_state.keys())[:3] if opt_state else []
    if opt_state:
        result["opt_steps"] = sorted({int(float(st["step"])) for k, st in opt_state.items()
                                      if isinstance(st, dict) and "step" in st})
        sc = opt_state.get("__loss_scaler__")
        result["loss_scale"] = float(sc["scale"]) if sc else None
    result["split_points"] = [list(m.plan.split_points) for m in runner.modules
                              if m.plan is not None]
    result["state_dict_keys"] = len(model.state_dict())
    w = getattr(runner, "worker", None)
    result["graphs"] = sum(1 for g in getattr(w, "graphs", {}).values() if not g.failed)
    result["graphs_failed"] = sum(1 for g in getattr(w, "graphs", {}).values() if g.failed)
    if state.dp_size > 1:
        # replicas must hold identical parameters after training
        flat = torch.cat([p.detach().cpu().reshape(-1) for p in model.parameters()])
        result["param_checksum"] = float(flat.double().sum())
    if state.is_main_process or state.dp_size > 1:
        path = args.out if state.is_main_process else f"{args.out}.dp{state.dp_rank}"
        with open(path, "w") as f:
            json.dump(result, f)
    runner.close()


if __name__ == "__main__":
    main()
