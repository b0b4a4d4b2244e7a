"""Thin tensor-level wrappers over the C ABI of the kernel library (no autograd here).

Each function validates shapes, allocates outputs with torch (so memory comes from the caching
allocator of the current stream) and launches on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import c_f, c_ll, check, dt, ptr, sm_count, stream

# GEMM epilogue codes (gemm_sm100.cu)
EPI_NONE, EPI_GELU, EPI_DGELU, EPI_GELU_TANH, EPI_DGELU_TANH, EPI_SILU = 0, 1, 2, 3, 4, 5
# elementwise op codes (elementwise.cu)
EW_GELU, EW_GELU_TANH, EW_SILU, EW_COPY = 0, 1, 2, 3
EW_DGELU, EW_DGELU_TANH, EW_DSILU = 10, 11, 12
EW_ADD, EW_MUL, EW_SILU_MUL, EW_GELU_MUL = 20, 21, 30, 31

_status = {}
_status_host = {}
STATUS_WORDS = 4     # [0] first error code, [1] wait limit in 1024-cycle units (0 = built-in)
_STATUS_NAMES = {1: "TIMEOUT_FULL", 2: "TIMEOUT_EMPTY", 3: "TIMEOUT_TMEM_FULL",
                 4: "TIMEOUT_TMEM_EMPTY", 5: "TIMEOUT_PEER_FLAG", 6: "BAD_ARG"}
PF_ERR_TIMEOUT_PEER_FLAG = 5


def status_word(device=None) -> torch.Tensor:
    """int32[STATUS_WORDS] per device.  Kernels record the first bounded-wait failure in word 0
    (0 = ok) and read their wait limit from word 1 (``set_wait_limit``); the environment
    variable PF_WAIT_CYCLES presets that limit."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx not in _status:
        t = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=f"cuda:{idx}")
        import os
        env = os.environ.get("PF_WAIT_CYCLES")
        if env:
            t[1] = max(1, int(float(env)) >> 10)
        _status[idx] = t
    return _status[idx]


def set_wait_limit(cycles: Optional[int], device=None) -> None:
    """Bounds every in-kernel wait (mbarrier, peer flag) to about `cycles` SM clock cycles;
    None restores the built-in limit (about a second)."""
    status_word(device)[1] = 0 if not cycles else max(1, int(cycles) >> 10)


def _raise_status(code: int) -> None:
    raise _lib.KernelError(f"a kernel reported status {code} "
                           f"({_STATUS_NAMES.get(code, '?')}: a bounded wait ran out)")


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises if any kernel gave up on a wait."""
    code = int(status_word(device)[0].item())
    if code != 0:
        status_word(device)[0] = 0
        _raise_status(code)


def poll_status(device=None) -> None:
    """The same check without stalling the host: every call raises if the copy started by the
    PREVIOUS call shows a failure, then starts a new asynchronous copy of the status word to
    pinned memory on the current stream.  Called once per training step, it reports a kernel
    that gave up on a wait one step later."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    ent = _status_host.get(idx)
    if ent is None:
        ent = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
        _status_host[idx] = ent
    if ent["event"] is not None:
        ent["event"].synchronize()       # recorded a whole step ago: long since complete
        code = int(ent["host"][0])
        if code != 0:
            ent["event"] = None
            status_word(idx)[0] = 0
            _raise_status(code)
    ent["host"].copy_(status_word(idx)[:1], non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(idx))
    ent["event"] = ev


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         aux: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE, accumulate: bool = False,
         alpha: float = 1.0, tile_n: int = 0) -> torch.Tensor:
    """out[M,N] = epi(alpha * A . B^T).

    a: [M,K] (K-major) or [K,M] when ``a_mn``; b: [N,K] (K-major) or [K,N] when ``b_mn``.
    Inputs are fp16 or bf16 2-D tensors with unit inner stride and 16-byte aligned pitch.
    """
    L = _lib.lib()
    assert a.dim() == 2 and b.dim() == 2 and a.dtype == b.dtype
    assert a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if residual is not None:
        assert residual.shape == (M, N) and residual.dtype == out.dtype and residual.stride(1) == 1
    if aux is not None:
        assert aux.shape == (M, N) and aux.dtype == out.dtype and aux.stride(1) == 1
    code = L.pf_gemm(ptr(a), ptr(b), ptr(out), M, N, K, c_ll(a.stride(0)), c_ll(b.stride(0)),
                     c_ll(out.stride(0)), int(a_mn), int(b_mn), dt(a.dtype), dt(out.dtype),
                     ptr(bias), dt(bias.dtype) if bias is not None else 0, ptr(residual),
                     c_ll(residual.stride(0) if residual is not None else 0), ptr(aux),
                     c_ll(aux.stride(0) if aux is not None else 0), epilogue, int(accumulate),
                     c_f(alpha), ptr(status_word(a.device)), sm_count(a.device), tile_n, stream())
    if code != 0:
        check(code, f"pf_gemm(M={M}, N={N}, K={K}, a={tuple(a.shape)}/{a.stride()}/{a.dtype}/"
                    f"{a.data_ptr() % 256}, b={tuple(b.shape)}/{b.stride()}/{b.data_ptr() % 256}, "
                    f"a_mn={a_mn}, b_mn={b_mn}, out={out.dtype}/{out.stride()})")
    check(code, "pf_gemm")
    return out


def elementwise(op: int, a: torch.Tensor, b: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    L = _lib.lib()
    a = a.contiguous()
    if b is not None:
        b = b.contiguous()
        assert b.shape == a.shape and b.dtype == a.dtype
    if out is None:
        out = torch.empty_like(a)
    check(L.pf_elementwise(ptr(a), ptr(b), ptr(out), c_ll(a.numel()), op, dt(a.dtype),
                           sm_count(a.device), stream()), "pf_elementwise")
    return out


def glu_fwd(gu: torch.Tensor, gelu: bool) -> torch.Tensor:
    L = _lib.lib()
    gu = gu.contiguous()
    H = gu.shape[-1] // 2
    out = torch.empty(gu.shape[:-1] + (H,), dtype=gu.dtype, device=gu.device)
    rows = gu.numel() // (2 * H)
    check(L.pf_glu_fwd(ptr(gu), ptr(out), c_ll(rows), H, int(gelu), dt(gu.dtype),
                       sm_count(gu.device), stream()), "pf_glu_fwd")
    return out


def glu_bwd(gu: torch.Tensor, dout: torch.Tensor, gelu: bool) -> torch.Tensor:
    L = _lib.lib()
    gu = gu.contiguous()
    dout = dout.contiguous()
    H = gu.shape[-1] // 2
    dgu = torch.empty_like(gu)
    rows = gu.numel() // (2 * H)
    check(L.pf_glu_bwd(ptr(gu), ptr(dout), ptr(dgu), c_ll(rows), H, int(gelu), dt(gu.dtype),
                       sm_count(gu.device), stream()), "pf_glu_bwd")
    return dgu


def axpy_f32(dst: torch.Tensor, src: torch.Tensor, scale: float = 1.0,
             accumulate: bool = True) -> torch.Tensor:
    L = _lib.lib()
    assert dst.dtype == torch.float32 and dst.is_contiguous() and dst.numel() == src.numel()
    src = src.contiguous()
    check(L.pf_axpy_f32(ptr(dst), ptr(src), c_ll(src.numel()), c_f(scale), int(accumulate),
                        dt(src.dtype), sm_count(src.device), stream()), "pf_axpy_f32")
    return dst


def cast(src: torch.Tensor, dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    L = _lib.lib()
    src = src.contiguous()
    if out is None:
        out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(L.pf_cast(ptr(src), ptr(out), c_ll(src.numel()), dt(src.dtype), dt(dtype),
                    sm_count(src.device), stream()), "pf_cast")
    return out


def colsum(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[c] += sum over rows of x[r, c]; ``out`` fp32, zero-filled when not given."""
    L = _lib.lib()
    assert x.dim() == 2 and x.stride(1) == 1
    if out is None:
        out = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
    check(L.pf_colsum(ptr(x), ptr(out), c_ll(x.shape[0]), x.shape[1], c_ll(x.stride(0)),
                      dt(x.dtype), sm_count(x.device), stream()), "pf_colsum")
    return out


def transpose16(x: torch.Tensor) -> torch.Tensor:
    L = _lib.lib()
    assert x.dim() == 2 and x.element_size() == 2 and x.stride(1) == 1
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    check(L.pf_transpose16(ptr(x), ptr(out), x.shape[0], x.shape[1], c_ll(x.stride(0)),
                           c_ll(out.stride(0)), stream()), "pf_transpose16")
    return out


def norm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
             rms: bool, residual: Optional[torch.Tensor] = None
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (y, h, mean, rstd); h = x + residual (h is x itself when residual is None)."""
    L = _lib.lib()
    N = x.shape[-1]
    x2 = x.contiguous().view(-1, N)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    res2 = residual.contiguous().view(-1, N) if residual is not None else None
    h = torch.empty_like(x2) if residual is not None else x2
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    g = gamma if gamma.dtype == torch.float32 else gamma.float()
    b = None if beta is None else (beta if beta.dtype == torch.float32 else beta.float())
    check(L.pf_norm_fwd(ptr(x2), ptr(res2), ptr(g), ptr(b), ptr(y),
                        ptr(h) if residual is not None else ptr(None), ptr(mean), ptr(rstd),
                        c_ll(rows), N, c_f(eps), int(rms), dt(x.dtype), stream()), "pf_norm_fwd")
    return y.view(x.shape), h.view(x.shape), mean, rstd


def norm_bwd_scratch_shape(rows: int, N: int, device=None) -> Tuple[int, int, int]:
    L = _lib.lib()
    return (L.pf_norm_bwd_ctas(c_ll(rows), sm_count(device)), 2, N)


def norm_bwd(dy: torch.Tensor, h: torch.Tensor, gamma: torch.Tensor, mean: torch.Tensor,
             rstd: torch.Tensor, rms: bool, dres: Optional[torch.Tensor] = None,
             dgamma: Optional[torch.Tensor] = None, dbeta: Optional[torch.Tensor] = None,
             accumulate: bool = False, want_dbeta: bool = True
             ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    L = _lib.lib()
    N = h.shape[-1]
    dy2 = dy.contiguous().view(-1, N)
    h2 = h.contiguous().view(-1, N)
    rows = h2.shape[0]
    dres2 = dres.contiguous().view(-1, N) if dres is not None else None
    dx = torch.empty_like(h2)
    g = gamma if gamma.dtype == torch.float32 else gamma.float()
    if dgamma is None:
        dgamma = torch.empty(N, dtype=torch.float32, device=h.device)
        accumulate = False
    if dbeta is None and want_dbeta and not rms:
        dbeta = torch.empty(N, dtype=torch.float32, device=h.device)
    scratch = torch.empty(norm_bwd_scratch_shape(rows, N, h.device), dtype=torch.float32,
                          device=h.device)
    check(L.pf_norm_bwd(ptr(dy2), ptr(h2), ptr(g), ptr(mean), ptr(rstd), ptr(dres2), ptr(dx),
                        ptr(dgamma), ptr(dbeta), ptr(scratch), c_ll(rows), N, int(rms),
                        int(accumulate), dt(h.dtype), sm_count(h.device), stream()), "pf_norm_bwd")
    return dx.view(h.shape), dgamma, dbeta


def nonfinite(g: torch.Tensor, found_inf: torch.Tensor) -> None:
    L = _lib.lib()
    assert g.dtype == torch.float32 and g.is_contiguous()
    check(L.pf_nonfinite(ptr(g), c_ll(g.numel()), ptr(found_inf), sm_count(g.device), stream()),
          "pf_nonfinite")


def adamw(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float,
          beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
          grad_scale: float = 1.0, decoupled: bool = True, zero_grad: bool = True,
          lp: Optional[torch.Tensor] = None, found_inf: Optional[torch.Tensor] = None,
          loss_scale: Optional[torch.Tensor] = None,
          applied_steps: Optional[torch.Tensor] = None) -> None:
    """`applied_steps` (int32 device scalar): when given, the bias correction uses its value + 1
    instead of `step`; advance it with ``step_advance`` after every group was updated."""
    L = _lib.lib()
    for t in (p, g, m, v):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == p.numel()
    check(L.pf_adamw(ptr(p), ptr(g), ptr(m), ptr(v), ptr(lp), c_ll(p.numel()), ptr(found_inf),
                     ptr(loss_scale), c_f(lr), c_f(beta1), c_f(beta2), c_f(eps),
                     c_f(weight_decay), int(step), ptr(applied_steps), c_f(grad_scale),
                     int(decoupled),
                     int(zero_grad), dt(lp.dtype) if lp is not None else 0, sm_count(p.device),
                     stream()), "pf_adamw")


def step_advance(applied_steps: torch.Tensor, found_inf: Optional[torch.Tensor]) -> None:
    """applied_steps += 1 unless `found_inf` is set (the step was skipped)."""
    L = _lib.lib()
    check(L.pf_step_advance(ptr(applied_steps), ptr(found_inf), stream()), "pf_step_advance")


def sgd(p: torch.Tensor, g: torch.Tensor, mom: Optional[torch.Tensor], *, lr: float,
        momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
        nesterov: bool = False, first_step: bool = False, grad_scale: float = 1.0,
        zero_grad: bool = True, lp: Optional[torch.Tensor] = None,
        found_inf: Optional[torch.Tensor] = None,
        loss_scale: Optional[torch.Tensor] = None) -> None:
    L = _lib.lib()
    check(L.pf_sgd(ptr(p), ptr(g), ptr(mom), ptr(lp), c_ll(p.numel()), ptr(found_inf),
                   ptr(loss_scale), c_f(lr), c_f(momentum), c_f(dampening), c_f(weight_decay),
                   int(nesterov), int(first_step), c_f(grad_scale), int(zero_grad),
                   dt(lp.dtype) if lp is not None else 0, sm_count(p.device), stream()), "pf_sgd")


def loss_scale_update(state: torch.Tensor, found_inf: torch.Tensor, growth: float = 2.0,
                      backoff: float = 0.5, interval: int = 2000) -> None:
    L = _lib.lib()
    check(L.pf_loss_scale_update(ptr(state), ptr(found_inf), c_f(growth), c_f(backoff),
                                 int(interval), stream()), "pf_loss_scale_update")


def ce_fwd(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100
           ) -> Tuple[torch.Tensor, torch.Tensor]:
    L = _lib.lib()
    assert logits.dim() == 2 and logits.stride(1) == 1 and target.dtype == torch.int64
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    check(L.pf_ce_fwd(ptr(logits), ptr(target.contiguous()), ptr(loss), ptr(lse), c_ll(rows), V,
                      c_ll(logits.stride(0)), c_ll(ignore_index), dt(logits.dtype), stream()),
          "pf_ce_fwd")
    return loss, lse


def ce_bwd(logits: torch.Tensor, target: torch.Tensor, lse: torch.Tensor,
           gscale: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    L = _lib.lib()
    rows, V = logits.shape
    d = torch.empty_like(logits)
    check(L.pf_ce_bwd(ptr(logits), ptr(target.contiguous()), ptr(lse), ptr(gscale), ptr(d),
                      c_ll(rows), V, c_ll(logits.stride(0)), c_ll(ignore_index),
                      dt(logits.dtype), stream()), "pf_ce_bwd")
    return d


def mse_fwd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    L = _lib.lib()
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty(1, dtype=torch.float32, device=a.device)
    check(L.pf_mse_fwd(ptr(a), ptr(b), ptr(out), c_ll(a.numel()), dt(a.dtype),
                       sm_count(a.device), stream()), "pf_mse_fwd")
    return out


def mse_bwd(a: torch.Tensor, b: torch.Tensor, gout: torch.Tensor) -> torch.Tensor:
    L = _lib.lib()
    a, b = a.contiguous(), b.contiguous()
    da = torch.empty_like(a)
    check(L.pf_mse_bwd(ptr(a), ptr(b), ptr(gout.float().contiguous()), ptr(da), c_ll(a.numel()),
                       dt(a.dtype), sm_count(a.device), stream()), "pf_mse_bwd")
    return da


def embed_fwd(table: torch.Tensor, ids: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    L = _lib.lib()
    ids_c = ids.contiguous()
    D = table.shape[1]
    out = torch.empty(ids.shape + (D,), dtype=out_dtype, device=table.device)
    check(L.pf_embed_fwd(ptr(table), ptr(ids_c), ptr(out), c_ll(ids_c.numel()), D,
                         c_ll(table.shape[0]), dt(table.dtype), dt(out_dtype), stream()),
          "pf_embed_fwd")
    return out


def embed_bwd(dout: torch.Tensor, ids: torch.Tensor, dtable: torch.Tensor) -> torch.Tensor:
    L = _lib.lib()
    assert dtable.dtype == torch.float32 and dtable.is_contiguous()
    dout = dout.contiguous()
    ids_c = ids.contiguous()
    check(L.pf_embed_bwd(ptr(dout), ptr(ids_c), ptr(dtable), c_ll(ids_c.numel()),
                         dtable.shape[1], c_ll(dtable.shape[0]), dt(dout.dtype), stream()),
          "pf_embed_bwd")
    return dtable


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False
         ) -> torch.Tensor:
    """x: [B, S, H, D] with unit stride on D; cos/sin: fp32 [S, D/2]."""
    L = _lib.lib()
    assert x.dim() == 4 and x.stride(3) == 1
    B, S, H, D = x.shape
    out = torch.empty((B, S, H, D), dtype=x.dtype, device=x.device)
    check(L.pf_rope(ptr(x), ptr(out), ptr(cos.contiguous()), ptr(sin.contiguous()), c_ll(B), S, H,
                    D, c_ll(x.stride(0)), c_ll(x.stride(1)), c_ll(x.stride(2)), int(inverse),
                    dt(x.dtype), sm_count(x.device), stream()), "pf_rope")
    return out


# --------------------------------------------------------------------------- attention
def attention_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """True when the native flash-attention kernels cover this problem."""
    L = _lib.lib()
    return L is not None and hasattr(L, "pf_attn_fwd") and _attn_ok(q, k, v)


def _attn_ok(q, k, v) -> bool:
    D = q.shape[-1]
    return (q.dtype in (torch.float16, torch.bfloat16) and D % 8 == 0 and D <= 128
            and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1)


def _strides3(t: torch.Tensor):
    return (ctypes.c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))


def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float
             ) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,Sq,H,D], k/v [B,Sk,H,D] (strided views allowed) -> (o [B,Sq,H,D], lse [B,H,Sq])."""
    L = _lib.lib()
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    fix = lambda t: t if (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and
                          all(s % 8 == 0 for s in t.stride()[:3])) else t.contiguous()
    q, k, v = fix(q), fix(k), fix(v)
    o = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    check(L.pf_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), B, H, Sq, Sk, D, _strides3(q),
                        _strides3(k), _strides3(v), int(causal), c_f(scale), dt(q.dtype),
                        ptr(status_word(q.device)), stream()), "pf_attn_fwd")
    return o, lse


def attn_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
             o: torch.Tensor, lse: torch.Tensor, causal: bool, scale: float,
             packed: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (dq, dk, dv).  With ``packed`` (self-attention on slices of one fused projection) the
    three gradients are slices of a single [B, S, 3, H, D] buffer, i.e. the gradient of the
    fused projection needs no concatenation."""
    L = _lib.lib()
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    fix = lambda t: t if (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and
                          all(s % 8 == 0 for s in t.stride()[:3])) else t.contiguous()
    q, k, v = fix(q), fix(k), fix(v)
    do, o = do.contiguous(), o.contiguous()
    if packed and Sq == Sk:
        dqkv = torch.empty((B, Sq, 3, H, D), dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    else:
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    acc = torch.empty((B, Sq, H, D), dtype=torch.float32, device=q.device)
    check(L.pf_attn_bwd(ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(delta), ptr(acc),
                        ptr(dq), ptr(dk), ptr(dv), B, H, Sq, Sk, D, _strides3(q), _strides3(k),
                        _strides3(v), _strides3(dq), _strides3(dk), int(causal), c_f(scale),
                        dt(q.dtype), ptr(status_word(q.device)), sm_count(q.device), stream()),
          "pf_attn_bwd")
    return dq, dk, dv


# --------------------------------------------------------------------------- UNet kernels (NHWC)
def im2col(x: torch.Tensor, KH: int, KW: int, stride: int, pad: int) -> torch.Tensor:
    L = _lib.lib()
    B, H, W, C = x.shape
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    cols = torch.empty((B * Ho * Wo, KH * KW * C), dtype=x.dtype, device=x.device)
    check(L.pf_im2col(ptr(x.contiguous()), ptr(cols), B, H, W, C, KH, KW, Ho, Wo, stride, pad,
                      c_ll(cols.stride(0)), dt(x.dtype), sm_count(x.device), stream()), "pf_im2col")
    return cols


def conv_gemm_supported(x: torch.Tensor, KH: int, KW: int, stride: int, pad: int) -> bool:
    """True when the implicit-GEMM convolution covers this problem: x NHWC with C % 64 == 0,
    tiles of 128 output pixels made of whole output rows of one image, stride 1 or 2."""
    B, H, W, C = x.shape
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    return (x.is_contiguous() and C % 64 == 0 and 0 < Wo <= 128 and 128 % Wo == 0
            and (Ho * Wo) % 128 == 0 and stride in (1, 2))


def conv_gemm(x: torch.Tensor, w2: torch.Tensor, KH: int, KW: int, stride: int, pad: int, *,
              bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
              epilogue: int = EPI_NONE) -> torch.Tensor:
    """Convolution as an implicit GEMM: x NHWC [B, H, W, C], w2 [Cout, KH*KW*C] (taps outermost,
    channels innermost) -> [B, Ho, Wo, Cout].  The patches are never materialised: the GEMM's A
    tiles come straight from x through a 4-D tensor map whose out-of-bounds fill is the zero
    padding."""
    L = _lib.lib()
    B, H, W, C = x.shape
    Cout = w2.shape[0]
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    assert w2.shape[1] == KH * KW * C and w2.stride(1) == 1 and w2.dtype == x.dtype
    y = torch.empty((B, Ho, Wo, Cout), dtype=x.dtype, device=x.device)
    r2 = residual.reshape(-1, Cout) if residual is not None else None
    check(L.pf_conv_gemm(ptr(x), ptr(w2), ptr(y), B, H, W, C, Cout, KH, KW, stride, pad,
                         c_ll(w2.stride(0)), c_ll(Cout), dt(x.dtype), dt(y.dtype), ptr(bias),
                         dt(bias.dtype) if bias is not None else 0, ptr(r2),
                         c_ll(r2.stride(0) if r2 is not None else 0), epilogue,
                         ptr(status_word(x.device)), sm_count(x.device), stream()),
          "pf_conv_gemm")
    return y


def conv_wgrad_supported(x: torch.Tensor, cout: int, KH: int, KW: int, stride: int, pad: int
                         ) -> bool:
    B, H, W, C = x.shape
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    return (x.is_contiguous() and C % 64 == 0 and cout % 8 == 0 and Wo > 0
            and (64 % Wo == 0 or Wo % 64 == 0) and (Ho * Wo) % 64 == 0 and stride in (1, 2))


def conv_wgrad(dy2: torch.Tensor, x: torch.Tensor, KH: int, KW: int, stride: int, pad: int,
               out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """dw2 [Cout, KH*KW*C] fp32 (+)= dy2[B*Ho*Wo, Cout]^T . patches(x) without an im2col buffer."""
    L = _lib.lib()
    B, H, W, C = x.shape
    Cout = dy2.shape[1]
    assert dy2.is_contiguous() and dy2.dtype == x.dtype
    if out is None:
        out = torch.empty((Cout, KH * KW * C), dtype=torch.float32, device=x.device)
        accumulate = False
    check(L.pf_conv_wgrad(ptr(dy2), ptr(x), ptr(out), B, H, W, C, Cout, KH, KW, stride, pad,
                          dt(x.dtype), int(accumulate), ptr(status_word(x.device)),
                          sm_count(x.device), stream()), "pf_conv_wgrad")
    return out


def col2im(dcols: torch.Tensor, shape, KH: int, KW: int, stride: int, pad: int) -> torch.Tensor:
    L = _lib.lib()
    B, H, W, C = shape
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    dx = torch.empty(shape, dtype=dcols.dtype, device=dcols.device)
    check(L.pf_col2im(ptr(dcols), ptr(dx), B, H, W, C, KH, KW, Ho, Wo, stride, pad,
                      c_ll(dcols.stride(0)), dt(dcols.dtype), sm_count(dcols.device), stream()),
          "pf_col2im")
    return dx


def groupnorm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, groups: int,
                  eps: float, silu: bool):
    """x NHWC [B, H, W, C] -> (y, mean[B*G], rstd[B*G])."""
    L = _lib.lib()
    x = x.contiguous()
    B, H, W, C = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(B * groups, dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    check(L.pf_groupnorm_fwd(ptr(x), ptr(gamma.float()), ptr(beta.float()), ptr(y), ptr(mean),
                             ptr(rstd), B, H * W, C, groups, c_f(eps), int(silu), dt(x.dtype),
                             sm_count(x.device), stream()), "pf_groupnorm_fwd")
    return y, mean, rstd


def groupnorm_bwd(dy, x, mean, rstd, gamma, beta, groups: int, silu: bool):
    L = _lib.lib()
    x, dy = x.contiguous(), dy.contiguous()
    B, H, W, C = x.shape
    dx = torch.empty_like(x)
    dgamma = torch.zeros(C, dtype=torch.float32, device=x.device)
    dbeta = torch.zeros(C, dtype=torch.float32, device=x.device)
    sums = torch.empty(2 * B * groups, dtype=torch.float32, device=x.device)
    check(L.pf_groupnorm_bwd(ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma.float()),
                             ptr(beta.float()), ptr(dx), ptr(dgamma), ptr(dbeta), ptr(sums), B,
                             H * W, C, groups, int(silu), dt(x.dtype), sm_count(x.device),
                             stream()), "pf_groupnorm_bwd")
    return dx, dgamma, dbeta


def upsample2x(x: torch.Tensor, backward: bool = False) -> torch.Tensor:
    L = _lib.lib()
    x = x.contiguous()
    B, H, W, C = x.shape
    if backward:
        H, W = H // 2, W // 2
        y = torch.empty((B, H, W, C), dtype=x.dtype, device=x.device)
    else:
        y = torch.empty((B, 2 * H, 2 * W, C), dtype=x.dtype, device=x.device)
    check(L.pf_upsample2x(ptr(x), ptr(y), B, H, W, C, int(backward), dt(x.dtype),
                          sm_count(x.device), stream()), "pf_upsample2x")
    return y


def gemm_allgather(a: torch.Tensor, w_full: torch.Tensor, copies_table, world: int, rank: int,
                   row_end, ready: torch.Tensor, *, bias=None, residual=None, aux=None,
                   epilogue: int = EPI_NONE, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = epi(a @ W^T) where the rows of W are owned by `world` ranks (rank r owns rows
    [row_end[r-1], row_end[r])); the kernel pulls the other ranks' rows into ``w_full`` over
    NVLink while it computes the tiles it already has.

    ``copies_table`` is a ctypes array with every rank's pointer to its full-size copy of W
    (peer-mapped, see ``parallel.dp_fused.PeerMemory.share``); a copy only has to be current in
    the rows its rank owns.  ``ready`` is an int32 tensor with one entry per 256-row tile of W
    plus one (the running total)."""
    L = _lib.lib()
    M, K = a.shape
    N = w_full.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    ends = (ctypes.c_int * world)(*[int(x) for x in row_end])
    check(L.pf_gemm_allgather(ptr(a), ptr(w_full), copies_table, world, rank, ends,
                              ptr(ready), ptr(out), M, N, K, c_ll(a.stride(0)),
                              c_ll(w_full.stride(0)), c_ll(out.stride(0)), dt(a.dtype),
                              dt(out.dtype), ptr(bias), dt(bias.dtype) if bias is not None else 0,
                              ptr(residual), c_ll(residual.stride(0) if residual is not None else 0),
                              ptr(aux), c_ll(aux.stride(0) if aux is not None else 0), epilogue,
                              c_f(1.0), ptr(status_word(a.device)), sm_count(a.device), stream()),
          "pf_gemm_allgather")
    return out


def gather_rows(w_full: torch.Tensor, copies_table, world: int, rank: int, row_end) -> None:
    """Copies the rows of a [rows, K] weight that other ranks own from their copies into
    ``w_full`` (stand-alone form of the gather, for first consumers that are not a GEMM)."""
    L = _lib.lib()
    assert w_full.dim() == 2 and w_full.is_contiguous()
    ends = (ctypes.c_int * world)(*[int(x) for x in row_end])
    check(L.pf_gather_rows(ptr(w_full), copies_table, ends, world, rank, w_full.shape[0],
                           c_ll(w_full.shape[1] * w_full.element_size()),
                           sm_count(w_full.device), stream()), "pf_gather_rows")
