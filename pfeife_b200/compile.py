"""Optional per-stage dynamo compilation (pfeife/compile.py:6-60): when ``option.compiler`` is
set each stage module is compiled with that backend on first use.  The native-kernel rewrite
is the default path; this hook exists for parity with ``--backend``."""
from __future__ import annotations

import torch


class WrapperModule(torch.nn.Module):
    def __init__(self, compiled, unwrap_singleton_tuple: bool):
        super().__init__()
        self.compiled = compiled
        self.unwrap = unwrap_singleton_tuple

    def forward(self, *args):
        out = self.compiled(*args)
        if self.unwrap and isinstance(out, (tuple, list)) and len(out) == 1:
            return out[0]
        return out


def compile_module(compiler, submod: torch.nn.Module, inputs=None) -> torch.nn.Module:
    if not compiler:
        return submod
    kwargs = {"mode": "max-autotune"} if compiler == "inductor" else {}
    compiled = torch.compile(submod, backend=compiler, **kwargs)
    return WrapperModule(compiled, unwrap_singleton_tuple=False)
