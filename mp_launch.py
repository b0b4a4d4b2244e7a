#!/usr/bin/env python
"""Launcher: starts ``world_size`` ranks and runs the user's training script on the main rank of
every pipeline and the worker loop on the others.

    python mp_launch.py --world_size 8 --dp_mesh "-2,4" train.py --batch_size 16 ...

Same CLI as the reference (mp_launch.py:14-46): ``--launcher {python,torchrun,slurm}
--world_size --nnodes --node_rank --all_main --dp_mesh --master_addr --master_port``, then the
script and its arguments.  The launcher re-enters itself once per rank with ``--run_proc``; a
rank is a *master* when it is the last pipeline rank of its pipeline (or always with
``--all_main``).  Ctrl-C terminates the children's process groups.
"""
from __future__ import annotations

import argparse
import os
import runpy
import signal
import subprocess
import sys
from typing import Dict, List

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--launcher", choices=["python", "torchrun", "slurm"], default="python")
    ap.add_argument("--world_size", type=int, default=1)
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node_rank", type=int, default=0)
    ap.add_argument("--all_main", action="store_true",
                    help="run the training script on every rank")
    ap.add_argument("--dp_mesh", type=str, default=None, help='e.g. "-2,4" (DP=2 x PP=4)')
    ap.add_argument("--master_addr", type=str, default="127.0.0.1")
    ap.add_argument("--master_port", type=str, default="24446")
    ap.add_argument("--cpu", action="store_true", help="gloo/CPU ranks (no GPU needed)")
    ap.add_argument("--run_proc", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("cmd", nargs=argparse.REMAINDER, help="training script and its arguments")
    return ap.parse_args(argv)


def base_env(args) -> Dict[str, str]:
    env = dict(os.environ)
    env.update(WORLD_SIZE=str(args.world_size), NNODES=str(args.nnodes),
               NODE_RANK=str(args.node_rank), MASTER_ADDR=args.master_addr,
               MASTER_PORT=str(args.master_port))
    if args.dp_mesh:
        env["DP_MESH"] = args.dp_mesh
    if args.cpu:
        env["PFEIFE_CPU"] = "1"
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    return env


def child_argv(args) -> List[str]:
    out = [os.path.abspath(__file__), "--run_proc", "--launcher", args.launcher,
           "--world_size", str(args.world_size), "--nnodes", str(args.nnodes),
           "--node_rank", str(args.node_rank)]
    if args.all_main:
        out.append("--all_main")
    if args.dp_mesh:
        out.append(f"--dp_mesh={args.dp_mesh}")   # "=": the value may start with "-"
    if args.cpu:
        out.append("--cpu")
    return out + ["--"] + [c for c in args.cmd if c != "--"]


def get_python_env(args, local_rank: int) -> Dict[str, str]:
    per_node = args.world_size // args.nnodes
    env = base_env(args)
    env.update(RANK=str(args.node_rank * per_node + local_rank), LOCAL_RANK=str(local_rank))
    return env


def get_slurm_env(args, e=None) -> Dict[str, str]:
    """Under ``srun`` every task derives its rank from SLURM's variables (read in the task
    itself: the launching process only has the batch step's own values)."""
    env = base_env(args)
    e = os.environ if e is None else e
    if "SLURM_PROCID" in e:
        env.update(RANK=e["SLURM_PROCID"], LOCAL_RANK=e.get("SLURM_LOCALID", "0"),
                   WORLD_SIZE=e.get("SLURM_NTASKS", str(args.world_size)),
                   NNODES=e.get("SLURM_NNODES", str(args.nnodes)),
                   NODE_RANK=e.get("SLURM_NODEID", str(args.node_rank)))
    return env


def init_main(args) -> int:
    per_node = args.world_size // max(1, args.nnodes)
    procs: List[subprocess.Popen] = []
    if args.launcher == "torchrun":
        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={args.nnodes}",
               f"--node-rank={args.node_rank}", f"--nproc-per-node={per_node}",
               "--master-addr", args.master_addr, "--master-port", str(args.master_port)]
        procs.append(subprocess.Popen(cmd + child_argv(args), env=base_env(args),
                                      start_new_session=True))
    elif args.launcher == "slurm":
        cmd = ["srun", sys.executable] + child_argv(args)
        env = base_env(args)
        for k in ("RANK", "LOCAL_RANK"):      # every task sets its own from SLURM_PROCID
            env.pop(k, None)
        procs.append(subprocess.Popen(cmd, env=env, start_new_session=True))
    else:
        for lr in range(per_node):
            procs.append(subprocess.Popen([sys.executable] + child_argv(args),
                                          env=get_python_env(args, lr), start_new_session=True))

    def kill_all(*_):
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass

    signal.signal(signal.SIGINT, lambda *_: (kill_all(), sys.exit(130)))
    signal.signal(signal.SIGTERM, lambda *_: (kill_all(), sys.exit(143)))
    rc = 0
    try:
        # a rank that dies takes the job down instead of leaving the others hanging
        remaining = list(procs)
        while remaining:
            for p in list(remaining):
                try:
                    r = p.wait(timeout=0.2)
                except subprocess.TimeoutExpired:
                    continue
                remaining.remove(p)
                if r != 0:
                    rc = rc or r
                    kill_all()
                    remaining = []
                    break
    finally:
        kill_all()
    return rc


def run_master(cmd: List[str]) -> None:
    """Runs the user's script in this process (``sys.argv`` = script + its arguments)."""
    script = cmd[0]
    sys.argv = [script] + cmd[1:]
    sys.path.insert(0, os.path.dirname(os.path.abspath(script)))
    runpy.run_path(script, run_name="__main__")


def run_worker() -> None:
    from pfeife_b200.runtime.partial import worker_loop
    from pfeife_b200.topology import initialize_pfeife
    initialize_pfeife()
    worker_loop()


def run_proc(args) -> None:
    from pfeife_b200.topology import check_main_rank
    if args.launcher == "slurm" and "SLURM_PROCID" in os.environ:
        os.environ.update(get_slurm_env(args))
    if args.dp_mesh:
        os.environ["DP_MESH"] = args.dp_mesh
    if args.cpu:
        os.environ["PFEIFE_CPU"] = "1"
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    cmd = [c for c in args.cmd if c != "--"]
    if args.all_main or check_main_rank(rank, world, os.environ.get("DP_MESH")):
        run_master(cmd)
    else:
        run_worker()


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.run_proc:
        run_proc(args)
        return 0
    if not args.cmd:
        print("mp_launch.py: no training script given", file=sys.stderr)
        return 2
    return init_main(args)


if __name__ == "__main__":
    sys.exit(main())
