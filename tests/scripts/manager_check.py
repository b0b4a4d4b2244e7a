"""Manager-style front-end (``PipeManager``: the framework owns loss and optimizer) run under
``mp_launch.py``: losses and parameters against a plain single-process loop, written to
``--out`` as JSON by the global main process."""
import argparse
import copy
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pfeife_b200 import PipeManager, PipeOption, initialize_pfeife  # noqa
from pfeife_b200.loss import CrossEntropyLoss  # noqa
from pfeife_b200.models.toy import DeepMLP  # noqa
from pfeife_b200.utils import set_seed  # noqa


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=3)
    PipeOption.add_arguments(ap)
    args = ap.parse_args()
    state = initialize_pfeife()
    option = PipeOption.from_args(args)
    set_seed(0)
    model = DeepMLP(16, 8, 10)
    ref = copy.deepcopy(model)
    model.to(state.device)
    manager = PipeManager(model, CrossEntropyLoss(10), option)
    ropt = option.make_optimizer(ref.parameters())
    n = option.batch_size * option.batch_cnt
    g = torch.Generator().manual_seed(5)
    losses, ref_losses = [], []
    for _ in range(args.steps):
        x, y = torch.randn(n, 16, generator=g), torch.randint(0, 10, (n,), generator=g)
        out = manager.run(y.to(state.device), x.to(state.device))
        losses.append([float(l) for l in out])
        ropt.zero_grad()
        cur = []
        for xm, ym in zip(x.chunk(option.batch_cnt), y.chunk(option.batch_cnt)):
            l = torch.nn.functional.cross_entropy(ref(xm), ym)
            l.backward()
            cur.append(float(l.detach()))
        ropt.step()
        ref_losses.append(cur)
    x = torch.randn(n, 16, generator=g)
    got = torch.cat([o.cpu() for o in manager.eval(x.to(state.device))])
    manager.gather_params()
    diff = max(float((p.detach().cpu() - q.detach()).abs().max())
               for p, q in zip(model.parameters(), ref.parameters()))
    with torch.no_grad():
        eval_diff = float((got - model.cpu()(x)).abs().max())
    manager.print_record()
    if state.is_main_process:
        with open(args.out, "w") as f:
            json.dump({"losses": losses, "ref_losses": ref_losses, "param_diff": diff,
                       "eval_diff": eval_diff}, f)
    manager.close()


if __name__ == "__main__":
    main()
