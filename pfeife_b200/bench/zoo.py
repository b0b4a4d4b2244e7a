"""Models for the benchmark drivers, by name (the reference's drivers load TorchBench and timm
models by name, benchmark_mp.py:158-184; neither package nor their weights exist offline, so
the names map to constructors that need no download).

``prepare_model(name, n)`` -> ``(model, args, kwargs, loss_fn)`` where ``args`` / ``kwargs`` hold
one optimizer step's worth of inputs (``n`` samples) and ``loss_fn(output, target, model)`` follows
the ``LossWrapper`` call shape.
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from ..loss import LossWrapper, MaskedLMOutputLoss, SumLoss


class TiedToy(torch.nn.Module):
    """Three 10x10 linear layers whose first and last share weight and bias: the smallest model
    in which two pipeline stages hold the same parameter (benchmark_mp.py:35-49)."""

    def __init__(self):
        super().__init__()
        self.linear = torch.nn.Linear(10, 10)
        self.linear2 = torch.nn.Linear(10, 10)
        self.linear3 = torch.nn.Linear(10, 10)
        self.linear.weight = self.linear3.weight
        self.linear.bias = self.linear3.bias

    def forward(self, x):
        return self.linear3(self.linear2(self.linear(x)))


def _hf(name: str, n: int):
    import transformers as tr
    small = dict(vocab_size=8192)
    table = {
        "hf_Bert": (tr.BertForMaskedLM, tr.BertConfig(**small), 128),
        "hf_Bert_large": (tr.BertForMaskedLM, tr.BertConfig(hidden_size=1024, num_hidden_layers=24,
                                                             num_attention_heads=16,
                                                             intermediate_size=4096, **small), 128),
        "hf_DistilBert": (tr.DistilBertForMaskedLM, tr.DistilBertConfig(**small), 128),
        "hf_Albert": (tr.AlbertForMaskedLM, tr.AlbertConfig(**small), 128),
        "hf_GPT2": (tr.GPT2LMHeadModel, tr.GPT2Config(**small), 256),
        "hf_GPT2_large": (tr.GPT2LMHeadModel, tr.GPT2Config(n_embd=1280, n_layer=36, n_head=20,
                                                            **small), 256),
        "hf_Roberta": (tr.RobertaForMaskedLM, tr.RobertaConfig(**small), 128),
    }
    if name not in table:
        raise ValueError(f"unknown model {name!r}; HuggingFace names: {sorted(table)}")
    cls, cfg, seq = table[name]
    for k in ("hidden_dropout_prob", "attention_probs_dropout_prob", "resid_pdrop", "embd_pdrop",
              "attn_pdrop", "dropout", "attention_dropout", "classifier_dropout_prob"):
        if hasattr(cfg, k):
            setattr(cfg, k, 0.0)          # the validity check compares against a second run
    ids = torch.randint(0, cfg.vocab_size, (n, seq))
    return cls(cfg), (), {"input_ids": ids, "labels": ids.clone()}, MaskedLMOutputLoss()


def _torchvision(name: str, n: int):
    import torchvision
    ctor = getattr(torchvision.models, name, None)
    if ctor is None:
        raise ValueError(f"torchvision has no model {name!r}")
    return ctor(num_classes=1000), (torch.rand(n, 3, 224, 224),), {}, SumLoss()


def _own(name: str, n: int):
    from .workloads import get_workload
    wl = get_workload(name)
    batch = wl.make_batch(n, torch.Generator().manual_seed(0))
    k = wl.n_model_inputs
    targets = batch[k:] if len(batch) > k else (batch[0],)     # language models: labels = ids

    class _Loss(LossWrapper):
        def forward(self, input, target=None, model=None):
            t = target if isinstance(target, (tuple, list)) else (target,)
            return wl.loss(lambda *a: input, *([None] * k), *t) if len(batch) > k else \
                wl.loss(lambda *a: input, *t)

    return wl.build_model(), tuple(batch[:k]), {}, _Loss(), targets


def prepare_model(name: str, n: int) -> Tuple[torch.nn.Module, tuple, Dict[str, Any], LossWrapper,
                                               Any]:
    """Returns ``(model, args, kwargs, loss_fn, target)``; ``target`` is None when the loss needs
    none (it is split into micro-batches with the inputs otherwise)."""
    if name == "toy":
        return TiedToy(), (torch.rand(n, 10),), {}, SumLoss(), None
    if name.startswith("hf_"):
        return (*_hf(name, n), None)
    if name.startswith("tv:") or name.startswith("torchvision:"):
        return (*_torchvision(name.split(":", 1)[1], n), None)
    if name.startswith("timm:"):
        try:
            import timm
        except ImportError as e:
            raise SystemExit("timm is not installed here; torchvision models are available as "
                             "tv:<name> (tv:resnet50, tv:vit_b_16, ...)") from e
        return timm.create_model(name[5:], pretrained=False), (torch.rand(n, 3, 224, 224),), {}, \
            SumLoss(), None
    from .workloads import WORKLOADS
    if name in WORKLOADS:
        model, args, kwargs, loss, targets = _own(name, n)
        return model, args, kwargs, loss, (targets if len(targets) > 1 else targets[0])
    raise ValueError(f"unknown model {name!r}: toy, hf_<Name>, tv:<name>, timm:<name> or one of "
                     f"{', '.join(WORKLOADS)}")


def replace_batch_norm(model: torch.nn.Module) -> torch.nn.Module:
    """Takes the batch-dependent and the random layers out, so that two runs of the same steps
    are comparable whatever the micro-batching (test/utils.py:206-229): BatchNorm becomes the
    identity; Dropout stays in place with probability 0 (code that reads ``.p`` keeps working)."""
    for name, child in list(model.named_children()):
        if isinstance(child, torch.nn.modules.batchnorm._BatchNorm):
            setattr(model, name, torch.nn.Identity())
        elif isinstance(child, torch.nn.modules.dropout._DropoutNd):
            child.p = 0.0
        else:
            replace_batch_norm(child)
    return model
