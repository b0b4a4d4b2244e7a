"""Llama-2-shaped decoder on the native ops (the reference trains HF ``LlamaForCausalLM`` with
eager attention, bench_models/models/train_llama.py:486-520).

Per layer: RMSNorm -> fused QKV GEMM -> RoPE on Q and K -> causal flash attention -> output
GEMM with the residual in its epilogue -> RMSNorm -> fused gate|up GEMM -> SwiGLU -> down GEMM
with the residual in its epilogue.  The score matrix is never materialised, which is what lets
the sequence-2048 configuration fit comfortably.  ``tie_embeddings`` shares the token embedding
with the LM head (a parameter used by the first and the last pipeline stage).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    max_seq_len: int = 2048
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_embeddings: bool = False


LLAMA_CONFIGS = {
    "llama2_7b": LlamaConfig(),
    "llama_tiny": LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_layers=4,
                              num_heads=4, max_seq_len=32),
}


def llama_config(name: str, **overrides) -> LlamaConfig:
    return LlamaConfig(**{**LLAMA_CONFIGS[name].__dict__, **overrides})


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d = cfg.hidden_size
        self.num_heads = cfg.num_heads
        self.eps = cfg.rms_eps
        self.input_norm = nn.Parameter(torch.ones(d))
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o_proj = nn.Linear(d, d, bias=False)
        self.post_norm = nn.Parameter(torch.ones(d))
        self.gate_up = nn.Linear(d, 2 * cfg.intermediate_size, bias=False)
        self.down = nn.Linear(cfg.intermediate_size, d, bias=False)

    def forward(self, x: torch.Tensor, delta, cos: torch.Tensor, sin: torch.Tensor):
        """(x, delta) -> (x', delta'): the residual stream is x + delta, summed inside the next
        RMSNorm launch so that every tensor of the stream has one consumer (its gradient is
        then complete when the norm's backward has added the part arriving through the sum)."""
        B, S, d = x.shape
        H = self.num_heads
        if delta is None:
            y = ops.rms_norm(x, self.input_norm, self.eps)
        else:
            y, x = ops.rms_norm(delta, self.input_norm, self.eps, residual=x)
        qkv = ops.linear(y, self.qkv.weight).view(B, S, 3, H, d // H)
        q = ops.rope(qkv[:, :, 0], cos, sin)
        k = ops.rope(qkv[:, :, 1], cos, sin)
        a = ops.attention(q, k, qkv[:, :, 2], causal=True).view(B, S, d)
        delta = ops.linear(a, self.o_proj.weight)
        y, x = ops.rms_norm(delta, self.post_norm, self.eps, residual=x)
        g = ops.swiglu(ops.linear(y, self.gate_up.weight))
        return x, ops.linear(g, self.down.weight)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([LlamaBlock(cfg) for _ in range(cfg.num_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size))
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed.weight
        cos, sin = ops.rope_tables(cfg.max_seq_len, cfg.hidden_size // cfg.num_heads,
                                   cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        S = input_ids.shape[1]
        x = ops.embedding(input_ids, self.embed.weight)
        cos, sin = self.rope_cos[:S], self.rope_sin[:S]
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, cos, sin)
        if delta is None:
            y = ops.rms_norm(x, self.norm, self.cfg.rms_eps)
        else:
            y, _ = ops.rms_norm(delta, self.norm, self.cfg.rms_eps, residual=x)
        return ops.linear(y, self.lm_head.weight)


def causal_lm_loss(logits: torch.Tensor, input_ids: torch.Tensor) -> torch.Tensor:
    """Next-token cross entropy (shift by one), fused log-softmax + NLL."""
    V = logits.shape[-1]
    return ops.cross_entropy(logits[:, :-1].reshape(-1, V), input_ids[:, 1:].reshape(-1))
