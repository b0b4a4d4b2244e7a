"""PipeOption: one flag table drives the constructor, argparse and ``from_args``
(the reference's flags, pfeife/option.py, plus this framework's own)."""
import argparse

from pfeife_b200 import PipeOption

REFERENCE_FLAGS = ["--backend", "--batch_cnt", "--batch_size", "--bench_seed", "--cpu",
                   "--device_bench", "--device_cnt", "--device_map", "--graph_bench",
                   "--linearizer", "--loop_batch", "--loop_cnt", "--mixed_precision",
                   "--no_bench_optimizer", "--no_io_cache", "--no_side_effect", "--old_ver",
                   "--optimizer_type", "--partitioner", "--prefetch_fwd", "--print_graph",
                   "--reducer_backend", "--scheduler", "--single_comm_thread", "--split_points",
                   "--use_fsdp", "--verbose"]


def _parser():
    ap = argparse.ArgumentParser()
    PipeOption.add_arguments(ap)
    return ap


def test_every_reference_flag_is_accepted():
    known = {s for a in _parser()._actions for s in a.option_strings}
    assert not [f for f in REFERENCE_FLAGS if f not in known]


def test_from_args_round_trip_and_defaults():
    args = _parser().parse_args(["--device_cnt", "4", "--batch_size", "8", "--batch_cnt", "6",
                                 "--loop_cnt", "2", "--prefetch_fwd", "1", "--mixed_precision",
                                 "bf16", "--use_fsdp", "--cuda_graphs", "--no_fused_dp"])
    opt = PipeOption.from_args(args)
    assert (opt.device_cnt, opt.batch_size, opt.batch_cnt, opt.loop_cnt, opt.prefetch_fwd) == \
        (4, 8, 6, 2, 1)
    assert str(opt.mixed_precision).endswith("bfloat16") or opt.mixed_precision == "bf16"
    assert opt.use_fsdp and opt.cuda_graphs and not opt.fused_dp
    d = opt.to_dict()
    assert d["device_cnt"] == 4 and d["use_fsdp"] is True
    # The command line and the constructor have the reference's (different) defaults for three
    # fields (pfeife/option.py:58-59 against :115 and :186-187); everything else agrees.
    dflt = PipeOption.from_args(_parser().parse_args([])).to_dict()
    plain = PipeOption().to_dict()
    differing = {k for k in dflt if dflt[k] != plain[k]}
    assert differing == {"batch_size", "batch_cnt", "optimizer_kwargs"}
    assert (dflt["batch_size"], dflt["batch_cnt"], dflt["optimizer_kwargs"]["lr"]) == (2, 4, 1e-3)
    assert (plain["batch_size"], plain["batch_cnt"], plain["optimizer_kwargs"]["lr"]) == \
        (4, plain["device_cnt"], 1e-5)


def test_optimizer_spec_builds_the_named_optimizer():
    import torch
    opt = PipeOption(optimizer={"type": "adamw", "lr": 3e-4, "weight_decay": 0.1})
    o = opt.make_optimizer([torch.nn.Parameter(torch.zeros(2))])
    assert type(o).__name__ == "AdamW" and o.param_groups[0]["lr"] == 3e-4
