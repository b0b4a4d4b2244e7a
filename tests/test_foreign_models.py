"""Models the framework did not write: HuggingFace transformers and a torchvision ResNet go
through capture, planning, partitioning and the pipelined runtime unchanged, and train like the
un-pipelined module (same micro-batches, same optimizer).  CPU threads, two stages."""
import copy

import pytest
import torch

from pfeife_b200 import PipeOption
from pfeife_b200.loss import MaskedLMOutputLoss, SumLoss
from pfeife_b200.runtime.manager import LocalPipeManager

BATCH_CNT, MICRO = 4, 2


def _bert():
    tr = pytest.importorskip("transformers")
    cfg = tr.BertConfig(hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                        intermediate_size=128, vocab_size=512, max_position_embeddings=64,
                        hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    ids = torch.randint(0, 512, (BATCH_CNT * MICRO, 16))
    return tr.BertForMaskedLM(cfg), {"input_ids": ids, "labels": ids.clone()}, MaskedLMOutputLoss()


def _gpt2():
    tr = pytest.importorskip("transformers")
    cfg = tr.GPT2Config(n_embd=64, n_layer=4, n_head=4, vocab_size=512, n_positions=64,
                        resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    ids = torch.randint(0, 512, (BATCH_CNT * MICRO, 16))
    # GPT-2 ties the output projection to the token embedding: with two stages the tensor lives
    # on both and its gradient is summed across them before the step
    return tr.GPT2LMHeadModel(cfg), {"input_ids": ids, "labels": ids.clone()}, MaskedLMOutputLoss()


def _resnet():
    tv = pytest.importorskip("torchvision")
    # BatchNorm buffers are updated in the forward pass and ReLU overwrites its input
    return tv.models.resnet18(num_classes=10), {"x": torch.randn(BATCH_CNT * MICRO, 3, 64, 64)}, \
        SumLoss()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("build", [_bert, _gpt2, _resnet], ids=["hf_bert", "hf_gpt2", "resnet18"])
def test_foreign_model_trains_like_the_unpipelined_module(build):
    torch.manual_seed(0)
    model, kwargs, loss_fn = build()
    model.train()
    ref = copy.deepcopy(model)
    option = PipeOption(device_cnt=2, batch_size=MICRO, batch_cnt=BATCH_CNT, cpu_test=True,
                        no_bench_optimizer=True, optimizer={"type": "adam", "lr": 1e-3})
    mgr = LocalPipeManager(model, loss_fn, option)
    ropt = torch.optim.Adam(ref.parameters(), lr=1e-3)
    try:
        for step in range(3):
            got = [float(l) for l in mgr.run(None, **kwargs)]
            ropt.zero_grad()
            want = []
            for mb in range(BATCH_CNT):
                sl = slice(mb * MICRO, (mb + 1) * MICRO)
                out = ref(**{k: v[sl] for k, v in kwargs.items()})
                loss = loss_fn(out, None, ref)
                loss.backward()
                want.append(float(loss.detach()))
            ropt.step()
            assert got == pytest.approx(want, rel=2e-3, abs=2e-3), (step, got, want)
        assert len(mgr.runner.modules[0].part.stages) >= 2
        mgr.gather_params()
        for (k, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.detach().cpu(), q.detach(), rtol=2e-3, atol=2e-4), k
        # buffers the forward pass updates (BatchNorm statistics and step counts) come back too
        for (k, b), (_, c) in zip(model.named_buffers(), ref.named_buffers()):
            assert torch.allclose(b.detach().cpu().float(), c.detach().float(), rtol=2e-3,
                                  atol=2e-4), k
    finally:
        mgr.close()
