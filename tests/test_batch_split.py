"""Micro-batch splitting of call arguments (the contract of pfeife/batch.py:30-132)."""
import torch

from pfeife_b200.utils.batch import split_args_kwargs


def test_tensors_split_on_dim0_lists_are_sliced_everything_else_is_replicated():
    x = torch.arange(24.).view(6, 4)
    mask = torch.ones(6, 2)
    names = ["a", "b", "c", "d", "e", "f"]
    args, kwargs = split_args_kwargs((x, {"mask": mask, "flag": True}, names, 7),
                                     {"labels": torch.arange(6), "scale": torch.tensor(2.0)}, 3)
    assert len(args) == len(kwargs) == 3
    for i, (a, k) in enumerate(zip(args, kwargs)):
        assert torch.equal(a[0], x[2 * i:2 * i + 2])
        assert torch.equal(a[1]["mask"], mask[2 * i:2 * i + 2]) and a[1]["flag"] is True
        assert a[2] == names[2 * i:2 * i + 2] and a[3] == 7
        assert torch.equal(k["labels"], torch.arange(6)[2 * i:2 * i + 2])
        assert float(k["scale"]) == 2.0          # a 0-dim tensor is replicated


def test_uneven_split_follows_tensor_split_and_nested_tensors_are_reached():
    x = torch.arange(7)
    args, _ = split_args_kwargs(([x, (x * 2, "tag")],), None, 3)
    sizes = [a[0][0].numel() for a in args]
    assert sizes == [3, 2, 2]
    assert torch.equal(torch.cat([a[0][1][0] for a in args]), x * 2)
    assert all(a[0][1][1] == "tag" for a in args)


def test_call_without_positional_arguments():
    args, kwargs = split_args_kwargs(None, {"x": torch.zeros(4, 1)}, 2)
    assert args == [(None,), (None,)] and kwargs[1]["x"].shape == (2, 1)
