"""Differentiable ops backed by the sm_100a kernels.

Every op is a ``torch.library`` custom op (opaque to dynamo, so captured stage graphs carry it
as one node) with
  * a CUDA implementation that calls the native kernels (no eager fallback on GPU for 16-bit
    tensors; fp32 tensors on CUDA, which no benchmark configuration uses, take the ATen path),
  * a CPU implementation in plain PyTorch, which is the numerical oracle of the tests and what
    the CPU/gloo pipeline tests execute,
  * a shape-only fake implementation, and
  * an autograd formula whose backward is again a custom op.

Mixed precision: parameters stay fp32 ("master"); ``register_param`` attaches a 16-bit shadow
and an fp32 gradient-bucket view to a master tensor.  ``linear`` then reads the shadow, and its
wgrad GEMM accumulates straight into the bucket from the epilogue (returning no autograd
gradient for the weight), which is what the fused data-parallel reduce consumes.
"""
from __future__ import annotations

import contextlib
import math
import threading
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor
from torch._subclasses.fake_tensor import FakeTensor

from . import kernels as kx

ACT_NONE, ACT_GELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3
_ACT_NAMES = {None: 0, "none": 0, "gelu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2, "silu": 3}


# --------------------------------------------------------------------------- parameter registry
@dataclass
class ParamSlot:
    lp: Optional[Tensor] = None          # 16-bit shadow of the master weight
    main_grad: Optional[Tensor] = None   # fp32 view into the flat gradient bucket
    # Deferred all-gather (sharded data parallelism): after an optimizer step only the rows this
    # rank owns are current in `lp`; the first consumer pulls the other rows from their owners.
    gather: Optional["GatherInfo"] = None
    gathered_in: int = 0                 # gather session that last completed `lp`


@dataclass
class GatherInfo:
    copies: object                       # ctypes array: every rank's pointer to its copy of lp
    row_end: Tuple[int, ...]             # rank r owns rows [row_end[r-1], row_end[r])
    world: int
    rank: int
    ready: Tensor                        # int32 scratch: one counter per 256-row tile + 1


_PARAMS: Dict[int, ParamSlot] = {}


def register_param(master: Tensor, lp: Optional[Tensor] = None,
                   main_grad: Optional[Tensor] = None) -> None:
    slot = ParamSlot(lp, main_grad)
    _PARAMS[master.data_ptr()] = slot
    if lp is not None:
        _PARAMS[lp.data_ptr()] = slot


def unregister_params() -> None:
    _PARAMS.clear()


# Gather sessions.  The runtime knows when a stage runs its first forward after an optimizer step
# (the only time its row-sharded weights are incomplete) and brackets that forward with
# ``gather_session(True)`` ... ``gather_session(False)``: inside, the first consumer of each
# sharded weight gathers it; outside, weights are taken as complete.  Keeping this decision out
# of per-weight state makes a captured CUDA graph of that forward replay the same gathers.
_session_tls = threading.local()
_session_counter = [0]


def gather_session(active: bool) -> None:
    if active:
        _session_counter[0] += 1
        _session_tls.id = _session_counter[0]
    else:
        _session_tls.id = 0


def set_gather(master: Tensor, info: GatherInfo) -> None:
    """Marks the registered parameter `master` as row-sharded between optimizer steps."""
    _PARAMS[master.data_ptr()].gather = info


def _stale(slot: Optional[ParamSlot]) -> bool:
    sid = getattr(_session_tls, "id", 0)
    return slot is not None and slot.gather is not None and sid != 0 and slot.gathered_in != sid


def _gather_now(slot: ParamSlot) -> None:
    """Stand-alone gather of the other ranks' rows (first consumer is not the fused GEMM)."""
    g = slot.gather
    kx.gather_rows(slot.lp.view(slot.lp.shape[0], -1), g.copies, g.world, g.rank, g.row_end)
    slot.gathered_in = _session_tls.id


def _slot(t: Tensor) -> Optional[ParamSlot]:
    return _PARAMS.get(t.data_ptr())


def _grad_bucket(t: Optional[Tensor]) -> Optional[Tensor]:
    """The flat fp32 gradient view registered for parameter `t` (bias, norm weight), or None.
    Backward kernels add into it directly, which saves the temporary, its zero-fill and the
    accumulation kernel autograd would launch."""
    if t is None or not t.is_cuda:
        return None
    s = _slot(t)
    if s is None or s.main_grad is None or s.main_grad.dtype != torch.float32 \
            or s.main_grad.numel() != t.numel():
        return None
    return s.main_grad.view(-1)


_trace_tls = threading.local()


@contextlib.contextmanager
def stage_precision(dtype: Optional[torch.dtype]):
    """Declares the autocast dtype the stages will run in, for the time a graph is traced.
    Shape-and-dtype inference of a trace runs the ops' meta functions with autocast switched
    off, so they would report x's dtype where the real op returns the autocast dtype, and a
    ``t.to(y.dtype)`` in the model would be baked into the graph with the wrong type."""
    prev = getattr(_trace_tls, "dtype", None)
    _trace_tls.dtype = dtype
    try:
        yield
    finally:
        _trace_tls.dtype = prev


def compute_dtype(x: Tensor) -> torch.dtype:
    """dtype GEMM-like ops run in: the autocast dtype when autocast is on (or, while a graph is
    traced, the one declared by ``stage_precision``), else x's dtype."""
    dev = "cuda" if x.is_cuda else "cpu"
    if torch.is_autocast_enabled(dev):
        return torch.get_autocast_dtype(dev)
    hint = getattr(_trace_tls, "dtype", None)
    if hint is not None and isinstance(x, FakeTensor):
        return hint
    return x.dtype


def _weight_as(w: Tensor, dtype: torch.dtype) -> Tensor:
    """`w` in `dtype`: itself, its registered 16-bit shadow, or a cast copy."""
    if w.dtype == dtype:
        return w
    s = _slot(w)
    if s is not None and s.lp is not None and s.lp.dtype == dtype:
        if _stale(s):
            _gather_now(s)
        return s.lp
    return kx.cast(w, dtype) if w.is_cuda else w.to(dtype)


def _native(x: Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.float16, torch.bfloat16)


def _act_ref(z: Tensor, act: int) -> Tensor:
    if act == ACT_GELU:
        return F.gelu(z)
    if act == ACT_GELU_TANH:
        return F.gelu(z, approximate="tanh")
    if act == ACT_SILU:
        return F.silu(z)
    return z


def _dact_ref(z: Tensor, act: int) -> Tensor:
    """Closed-form activation derivative in fp32 (autograd is unavailable inside an op)."""
    x = z.detach().float()
    if act == ACT_GELU:
        cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
        pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
        return cdf + x * pdf
    if act == ACT_GELU_TANH:
        u = 0.7978845608028654 * (x + 0.044715 * x ** 3)
        t = torch.tanh(u)
        du = 0.7978845608028654 * (1.0 + 3 * 0.044715 * x * x)
        return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * du
    if act == ACT_SILU:
        sg = torch.sigmoid(x)
        return sg * (1.0 + x * (1.0 - sg))
    return torch.ones_like(x)


def _pad_k(t: Tensor, mult: int = 8) -> Tensor:
    k = t.shape[-1]
    pad = (-k) % mult
    return F.pad(t, (0, pad)) if pad else t


def _rows(x: Tensor) -> Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    return x2


# =========================================================================== linear
@torch.library.custom_op("pfeife::linear_fwd", mutates_args=())
def linear_fwd(x: Tensor, w: Tensor, bias: Optional[Tensor], residual: Optional[Tensor],
               act: int) -> Tuple[Tensor, Tensor]:
    cd = compute_dtype(x)
    N = w.shape[0]
    out_shape = x.shape[:-1] + (N,)
    if x.is_cuda and cd in (torch.float16, torch.bfloat16):
        x2 = _rows(x if x.dtype == cd else kx.cast(x, cd))
        slot = _slot(w)
        fused_gather = _stale(slot) and slot.lp is not None and slot.lp.dtype == cd and \
            slot.lp.dim() == 2 and x2.shape[1] % 8 == 0
        w2 = slot.lp if fused_gather else _weight_as(w, cd)
        if x2.shape[1] % 8:
            x2, w2 = _pad_k(x2), _pad_k(w2)
        r2 = None
        if residual is not None:
            r2 = _rows(residual if residual.dtype == cd else kx.cast(residual, cd))
        M = x2.shape[0]
        y = torch.empty((M, N), dtype=cd, device=x.device)
        aux = torch.empty((M, N), dtype=cd, device=x.device) if act else None
        epi = {ACT_NONE: kx.EPI_NONE, ACT_GELU: kx.EPI_GELU, ACT_GELU_TANH: kx.EPI_GELU_TANH,
               ACT_SILU: kx.EPI_SILU}[act]
        if fused_gather:
            # first use of this weight since the optimizer step: the GEMM pulls the other
            # ranks' rows over NVLink while it computes the tiles whose rows are local
            g = slot.gather
            kx.gemm_allgather(x2, w2, g.copies, g.world, g.rank, g.row_end, g.ready, out=y,
                              bias=bias, residual=r2, aux=aux, epilogue=epi)
            slot.gathered_in = _session_tls.id
        else:
            kx.gemm(x2, w2, out=y, bias=bias, residual=r2, aux=aux, epilogue=epi)
        return y.view(out_shape), (aux.view(out_shape) if act else x.new_empty(0))
    # reference path (CPU, or fp32 on CUDA)
    xw = x.to(cd)
    z = F.linear(xw, w.to(cd), None if bias is None else bias.to(cd))
    y = _act_ref(z, act)
    if residual is not None:
        y = y + residual.to(cd)
    return y, (z if act else x.new_empty(0))


@linear_fwd.register_fake
def _(x, w, bias, residual, act):
    cd = compute_dtype(x)
    y = x.new_empty(x.shape[:-1] + (w.shape[0],), dtype=cd)
    return y, (torch.empty_like(y) if act else x.new_empty(0))


@torch.library.custom_op("pfeife::linear_bwd", mutates_args=())
def linear_bwd(dy: Tensor, x: Tensor, w: Tensor, aux: Tensor, act: int, need_dx: bool,
               need_dw: bool, need_db: bool, bias: Optional[Tensor] = None
               ) -> Tuple[Tensor, Tensor, Tensor]:
    """-> (dx, dw, db); an output that is not needed, or that was accumulated directly into a
    registered gradient bucket, comes back as an empty tensor."""
    cd = dy.dtype
    N, K = w.shape
    empty = dy.new_empty(0)
    slot = _slot(w)
    if dy.is_cuda and cd in (torch.float16, torch.bfloat16):
        dy2 = _rows(dy)
        if act:
            kop = {ACT_GELU: kx.EW_DGELU, ACT_GELU_TANH: kx.EW_DGELU_TANH, ACT_SILU: kx.EW_DSILU}[act]
            dy2 = kx.elementwise(kop, dy2, _rows(aux))
        dx, dw, db = dy.new_empty(0), dy.new_empty(0), dy.new_empty(0)
        if need_dx:
            w2 = _weight_as(w, cd)
            if N % 8 == 0 and K % 8 == 0:
                dx = kx.gemm(dy2, w2, b_mn=True).view(x.shape[:-1] + (K,))
            elif N % 8 == 0:
                dx = kx.gemm(dy2, _pad_k(w2), b_mn=True)[:, :K].reshape(x.shape[:-1] + (K,))
            else:
                dx = (dy2 @ w2).view(x.shape[:-1] + (K,))
        if need_dw:
            x2 = _rows(x if x.dtype == cd else kx.cast(x, cd))
            ok = N % 8 == 0 and K % 8 == 0
            if slot is not None and slot.main_grad is not None and ok:
                kx.gemm(dy2, x2, a_mn=True, b_mn=True, out=slot.main_grad.view(N, K),
                        accumulate=True)
            elif ok:
                dw = kx.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)
            elif N % 8 == 0:
                # input width not a multiple of 8 (ViT patch embedding: 3 * 14 * 14 = 588):
                # the same tensor-core GEMM on zero-padded columns, padding sliced off
                dw = kx.gemm(dy2, _pad_k(x2), a_mn=True, b_mn=True,
                             out_dtype=torch.float32)[:, :K].contiguous()
            else:
                dw = dy2.float().t() @ x2.float()
            if dw.numel() and w.dtype != torch.float32:
                dw = dw.to(w.dtype)
        if need_db:
            bucket = _grad_bucket(bias)
            if bucket is not None:
                kx.colsum(dy2, out=bucket)      # adds into the registered gradient
            else:
                db = kx.colsum(dy2)
        return dx, dw, db
    dz = dy if not act else (dy.float() * _dact_ref(aux, act)).to(cd)
    dz2 = dz.reshape(-1, N)
    dx = (dz2 @ w.to(cd)).view(x.shape[:-1] + (K,)) if need_dx else dy.new_empty(0)
    dw = (dz2.float().t() @ x.reshape(-1, K).float()).to(w.dtype) if need_dw else dy.new_empty(0)
    db = dz2.float().sum(0) if need_db else dy.new_empty(0)
    return dx, dw, db


@linear_bwd.register_fake
def _(dy, x, w, aux, act, need_dx, need_dw, need_db, bias=None):
    e = dy.new_empty(0)
    dx = dy.new_empty(x.shape[:-1] + (w.shape[1],)) if need_dx else e
    slot_acc = False
    dw = torch.empty_like(w) if need_dw and not slot_acc else e
    db = dy.new_empty(w.shape[0], dtype=torch.float32) if need_db else e
    return dx, dw, db


def _linear_setup(ctx, inputs, output):
    x, w, bias, residual, act = inputs
    y, aux = output
    ctx.set_materialize_grads(False)     # no zero tensor for the unused gradient of `aux`
    ctx.save_for_backward(x, w, aux, bias)
    ctx.act = act
    ctx.has_bias = bias is not None
    ctx.bias_dtype = bias.dtype if bias is not None else None
    ctx.has_res = residual is not None
    ctx.res_dtype = residual.dtype if residual is not None else None
    ctx.x_dtype = x.dtype


def _linear_backward(ctx, dy, daux):
    x, w, aux, bias = ctx.saved_tensors
    need = ctx.needs_input_grad
    if dy is None:
        return None, None, None, None, None
    dy = dy.contiguous()
    dx, dw, db = linear_bwd(dy, x, w, aux, ctx.act, need[0], need[1], ctx.has_bias and need[2],
                            bias)
    gx = dx.to(ctx.x_dtype) if need[0] else None
    gw = dw if (need[1] and dw.numel()) else None
    gb = db.to(ctx.bias_dtype) if (ctx.has_bias and need[2] and db.numel()) else None
    gr = dy.to(ctx.res_dtype) if (ctx.has_res and need[3]) else None
    return gx, gw, gb, gr, None


linear_fwd.register_autograd(_linear_backward, setup_context=_linear_setup)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
           activation: Optional[str] = None, residual: Optional[Tensor] = None) -> Tensor:
    """act(x @ weight.T + bias) + residual, one GEMM launch with a fused epilogue."""
    return linear_fwd(x, weight, bias, residual, _ACT_NAMES[activation])[0]


# =========================================================================== fused MLP
@torch.library.custom_op("pfeife::mlp_fwd", mutates_args=())
def mlp_fwd(x: Tensor, w1: Tensor, b1: Optional[Tensor], w2: Tensor, b2: Optional[Tensor],
            residual: Optional[Tensor], act: int) -> Tuple[Tensor, Tensor, Tensor]:
    """y = act(x W1^T + b1) W2^T + b2 (+ residual); also returns z1 (pre-activation) and a1."""
    a1, z1 = linear_fwd(x, w1, b1, None, act)
    y, _ = linear_fwd(a1, w2, b2, residual, ACT_NONE)
    return y, z1, a1


@mlp_fwd.register_fake
def _(x, w1, b1, w2, b2, residual, act):
    cd = compute_dtype(x)
    h = x.new_empty(x.shape[:-1] + (w1.shape[0],), dtype=cd)
    return x.new_empty(x.shape[:-1] + (w2.shape[0],), dtype=cd), h, torch.empty_like(h)


@torch.library.custom_op("pfeife::mlp_bwd", mutates_args=())
def mlp_bwd(dy: Tensor, x: Tensor, w1: Tensor, w2: Tensor, z1: Tensor, a1: Tensor, act: int,
            need_dx: bool, has_b1: bool, has_b2: bool, b1: Optional[Tensor] = None,
            b2: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """-> (dx, dw1, db1, dw2, db2).  On the native path the dgrad GEMM of the second layer
    applies act'(z1) in its epilogue, so dz1 is produced without an elementwise pass."""
    cd = dy.dtype
    empty = dy.new_empty(0)
    H, K = w1.shape
    N = w2.shape[0]
    if dy.is_cuda and cd in (torch.float16, torch.bfloat16) and act in (ACT_GELU, ACT_GELU_TANH) \
            and H % 8 == 0 and K % 8 == 0 and N % 8 == 0:
        dy2, z2, a2 = _rows(dy), _rows(z1), _rows(a1)
        w2c = _weight_as(w2, cd)
        epi = kx.EPI_DGELU if act == ACT_GELU else kx.EPI_DGELU_TANH
        dz1 = kx.gemm(dy2, w2c, b_mn=True, aux=z2, epilogue=epi)          # [M, H]
        _, dw2, db2 = linear_bwd(dy, a1, w2, empty, ACT_NONE, False, True, has_b2, b2)
        dx, dw1, db1 = linear_bwd(dz1.view(z1.shape), x, w1, empty, ACT_NONE, need_dx, True,
                                  has_b1, b1)
        return dx, dw1, db1, dw2, db2
    da1, dw2, db2 = linear_bwd(dy, a1, w2, empty, ACT_NONE, True, True, has_b2, b2)
    dx, dw1, db1 = linear_bwd(da1, x, w1, z1, act, need_dx, True, has_b1, b1)
    return dx, dw1, db1, dw2, db2


@mlp_bwd.register_fake
def _(dy, x, w1, w2, z1, a1, act, need_dx, has_b1, has_b2, b1=None, b2=None):
    e = dy.new_empty(0)
    f32 = torch.float32
    return (torch.empty_like(x, dtype=dy.dtype) if need_dx else e, torch.empty_like(w1),
            dy.new_empty(w1.shape[0], dtype=f32) if has_b1 else e, torch.empty_like(w2),
            dy.new_empty(w2.shape[0], dtype=f32) if has_b2 else e)


def _mlp_setup(ctx, inputs, output):
    x, w1, b1, w2, b2, residual, act = inputs
    y, z1, a1 = output
    ctx.set_materialize_grads(False)     # z1 / a1 are saved state, not differentiable outputs
    ctx.save_for_backward(x, w1, w2, z1, a1, b1, b2)
    ctx.act = act
    ctx.meta = (x.dtype, None if b1 is None else b1.dtype, None if b2 is None else b2.dtype,
                None if residual is None else residual.dtype)


def _mlp_backward(ctx, dy, dz1_unused, da1_unused):
    x, w1, w2, z1, a1, b1, b2 = ctx.saved_tensors
    xd, b1d, b2d, rd = ctx.meta
    need = ctx.needs_input_grad
    if dy is None:
        return (None,) * 7
    dy = dy.contiguous()
    dx, dw1, db1, dw2, db2 = mlp_bwd(dy, x, w1, w2, z1, a1, ctx.act, need[0], b1d is not None,
                                     b2d is not None, b1, b2)
    return (dx.to(xd) if need[0] else None,
            dw1 if dw1.numel() else None,
            db1.to(b1d) if (b1d is not None and db1.numel()) else None,
            dw2 if dw2.numel() else None,
            db2.to(b2d) if (b2d is not None and db2.numel()) else None,
            dy.to(rd) if (rd is not None and need[5]) else None,
            None)


mlp_fwd.register_autograd(_mlp_backward, setup_context=_mlp_setup)


def mlp(x: Tensor, w1: Tensor, b1: Optional[Tensor], w2: Tensor, b2: Optional[Tensor],
        activation: str = "gelu", residual: Optional[Tensor] = None) -> Tensor:
    """Transformer feed-forward block: two GEMMs, activation fused into the first epilogue,
    residual into the second, activation derivative into the dgrad epilogue."""
    return mlp_fwd(x, w1, b1, w2, b2, residual, _ACT_NAMES[activation])[0]


# =========================================================================== norms
@torch.library.custom_op("pfeife::norm_fwd", mutates_args=())
def norm_fwd(x: Tensor, gamma: Tensor, beta: Optional[Tensor], residual: Optional[Tensor],
             eps: float, rms: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """-> (y, h, mean, rstd) with h = x + residual (h aliases nothing: it is x's clone-free
    stand-in only on the fake/CPU path, always a fresh tensor when residual is given)."""
    N = x.shape[-1]
    if residual is not None and residual.dtype != x.dtype:
        residual = residual.to(x.dtype)      # the kernels read both streams as one type
    if _native(x) or (x.is_cuda and x.dtype == torch.float32 and N % 4 == 0):
        y, h, mean, rstd = kx.norm_fwd(x, gamma, beta, eps, rms, residual)
        if residual is None:
            h = x.new_empty(0)
        return y, h, mean, rstd
    hf = x.float() if residual is None else (x.float() + residual.float()).to(x.dtype).float()
    if rms:
        mean = hf.new_zeros(hf.shape[:-1]).reshape(-1)
        rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps).reshape(-1)
        y = hf * rstd.view(hf.shape[:-1] + (1,)) * gamma.float()
    else:
        mean = hf.mean(-1).reshape(-1)
        var = hf.var(-1, unbiased=False).reshape(-1)
        rstd = torch.rsqrt(var + eps)
        y = (hf - mean.view(hf.shape[:-1] + (1,))) * rstd.view(hf.shape[:-1] + (1,)) * gamma.float()
        if beta is not None:
            y = y + beta.float()
    h = hf.to(x.dtype) if residual is not None else x.new_empty(0)
    return y.to(x.dtype), h, mean, rstd


@norm_fwd.register_fake
def _(x, gamma, beta, residual, eps, rms):
    rows = x.numel() // x.shape[-1]
    st = x.new_empty(rows, dtype=torch.float32)
    return (torch.empty_like(x), torch.empty_like(x) if residual is not None else x.new_empty(0),
            st, torch.empty_like(st))


@torch.library.custom_op("pfeife::norm_bwd", mutates_args=())
def norm_bwd(dy: Tensor, dh: Optional[Tensor], h: Tensor, gamma: Tensor, mean: Tensor,
             rstd: Tensor, rms: bool, has_beta: bool, beta: Optional[Tensor] = None
             ) -> Tuple[Tensor, Tensor, Tensor]:
    """-> (dx [= dh_total], dgamma fp32, dbeta fp32).  `dh` is the gradient arriving through
    the residual-stream output, added in the same pass.  When gamma (and beta) have registered
    gradient buckets the sums are added there and come back empty."""
    N = h.shape[-1]
    if _native(h) or (h.is_cuda and h.dtype == torch.float32 and N % 4 == 0):
        e32 = dy.new_empty(0, dtype=torch.float32)
        gbucket = _grad_bucket(gamma)
        bbucket = _grad_bucket(beta) if has_beta else None
        if gbucket is not None and (bbucket is not None or not has_beta or rms):
            dx, _, _ = kx.norm_bwd(dy, h, gamma, mean, rstd, rms, dres=dh, dgamma=gbucket,
                                   dbeta=bbucket, accumulate=True, want_dbeta=False)
            return dx, e32, dy.new_empty(0, dtype=torch.float32)
        dx, dg, db = kx.norm_bwd(dy, h, gamma, mean, rstd, rms, dres=dh, want_dbeta=has_beta)
        return dx, dg, (db if (db is not None and has_beta) else e32)
    hf = h.float()
    shp = hf.shape[:-1] + (1,)
    xhat = (hf - (0 if rms else mean.view(shp))) * rstd.view(shp)
    dyf = dy.float()
    g = gamma.float()
    dyg = dyf * g
    m2 = (dyg * xhat).mean(-1, keepdim=True)
    m1 = 0 if rms else dyg.mean(-1, keepdim=True)
    dx = rstd.view(shp) * (dyg - m1 - xhat * m2)
    if dh is not None:
        dx = dx + dh.float()
    dg = (dyf * xhat).reshape(-1, N).sum(0)
    db = dyf.reshape(-1, N).sum(0) if has_beta else dy.new_empty(0, dtype=torch.float32)
    return dx.to(h.dtype), dg, db


@norm_bwd.register_fake
def _(dy, dh, h, gamma, mean, rstd, rms, has_beta, beta=None):
    N = h.shape[-1]
    return (torch.empty_like(h), h.new_empty(N, dtype=torch.float32),
            h.new_empty(N if has_beta else 0, dtype=torch.float32))


def _norm_setup(ctx, inputs, output):
    x, gamma, beta, residual, eps, rms = inputs
    y, h, mean, rstd = output
    ctx.set_materialize_grads(False)     # mean / rstd (and an unused h) carry no gradient
    ctx.save_for_backward(x if residual is None else h, gamma, mean, rstd, beta)
    ctx.rms = rms
    ctx.meta = (gamma.dtype, None if beta is None else beta.dtype, residual is not None,
                x.dtype, None if residual is None else residual.dtype)


def _norm_backward(ctx, dy, dh, dmean, drstd):
    h, gamma, mean, rstd, beta = ctx.saved_tensors
    gd, bd, has_res, xd, rd = ctx.meta
    dh_in = dh.contiguous() if (has_res and dh is not None) else None
    if dy is None:
        if dh_in is None:
            return (None,) * 6
        dy = torch.zeros_like(h)
    dx, dg, db = norm_bwd(dy.contiguous(), dh_in, h, gamma, mean, rstd, ctx.rms, bd is not None,
                          beta)
    return (dx.to(xd), dg.to(gd) if dg.numel() else None,
            db.to(bd) if (bd is not None and db.numel()) else None,
            dx.to(rd) if has_res else None, None, None)


norm_fwd.register_autograd(_norm_backward, setup_context=_norm_setup)


def layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float = 1e-5,
               residual: Optional[Tensor] = None):
    """LayerNorm over the last dim.  With ``residual`` returns ``(y, h)``, h = x + residual."""
    y, h, _, _ = norm_fwd(x, weight, bias, residual, eps, False)
    return (y, h) if residual is not None else y


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6, residual: Optional[Tensor] = None):
    y, h, _, _ = norm_fwd(x, weight, None, residual, eps, True)
    return (y, h) if residual is not None else y


# =========================================================================== activations
@torch.library.custom_op("pfeife::act_fwd", mutates_args=())
def act_fwd(x: Tensor, act: int) -> Tensor:
    if _native(x):
        op = {ACT_GELU: kx.EW_GELU, ACT_GELU_TANH: kx.EW_GELU_TANH, ACT_SILU: kx.EW_SILU}[act]
        return kx.elementwise(op, x).view(x.shape)
    return _act_ref(x, act)


@act_fwd.register_fake
def _(x, act):
    return torch.empty_like(x)


@torch.library.custom_op("pfeife::act_bwd", mutates_args=())
def act_bwd(dy: Tensor, x: Tensor, act: int) -> Tensor:
    if _native(x):
        op = {ACT_GELU: kx.EW_DGELU, ACT_GELU_TANH: kx.EW_DGELU_TANH, ACT_SILU: kx.EW_DSILU}[act]
        return kx.elementwise(op, dy.contiguous(), x).view(x.shape)
    return (dy.float() * _dact_ref(x, act)).to(x.dtype)


@act_bwd.register_fake
def _(dy, x, act):
    return torch.empty_like(x)


act_fwd.register_autograd(
    lambda ctx, dy: (act_bwd(dy, ctx.saved_tensors[0], ctx.act), None),
    setup_context=lambda ctx, inputs, output: (ctx.save_for_backward(inputs[0]),
                                               setattr(ctx, "act", inputs[1])))


def gelu(x: Tensor, approximate: str = "none") -> Tensor:
    return act_fwd(x, ACT_GELU_TANH if approximate == "tanh" else ACT_GELU)


def silu(x: Tensor) -> Tensor:
    return act_fwd(x, ACT_SILU)


@torch.library.custom_op("pfeife::glu_fwd", mutates_args=())
def glu_fwd(gu: Tensor, gelu_gate: bool) -> Tensor:
    if _native(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return kx.glu_fwd(gu, gelu_gate)
    H = gu.shape[-1] // 2
    g, u = gu[..., :H].float(), gu[..., H:].float()
    return ((F.gelu(g) if gelu_gate else F.silu(g)) * u).to(gu.dtype)


@glu_fwd.register_fake
def _(gu, gelu_gate):
    return gu.new_empty(gu.shape[:-1] + (gu.shape[-1] // 2,))


@torch.library.custom_op("pfeife::glu_bwd", mutates_args=())
def glu_bwd(dout: Tensor, gu: Tensor, gelu_gate: bool) -> Tensor:
    if _native(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return kx.glu_bwd(gu, dout, gelu_gate)
    H = gu.shape[-1] // 2
    g, u, d = gu[..., :H].float(), gu[..., H:].float(), dout.float()
    act = ACT_GELU if gelu_gate else ACT_SILU
    dg = d * u * _dact_ref(g, act)
    du = d * _act_ref(g, act)
    return torch.cat([dg, du], -1).to(gu.dtype)


@glu_bwd.register_fake
def _(dout, gu, gelu_gate):
    return torch.empty_like(gu)


glu_fwd.register_autograd(
    lambda ctx, dy: (glu_bwd(dy.contiguous(), ctx.saved_tensors[0], ctx.gelu_gate), None),
    setup_context=lambda ctx, inputs, output: (ctx.save_for_backward(inputs[0]),
                                               setattr(ctx, "gelu_gate", inputs[1])))


def swiglu(gate_up: Tensor) -> Tensor:
    """silu(gate) * up on a fused [..., 2H] projection (gate first)."""
    return glu_fwd(gate_up, False)


def geglu(gate_up: Tensor) -> Tensor:
    """gelu(gate) * up on a fused [..., 2H] projection (gate first)."""
    return glu_fwd(gate_up, True)


# =========================================================================== losses
@torch.library.custom_op("pfeife::ce_fwd", mutates_args=())
def ce_fwd(logits: Tensor, target: Tensor, ignore_index: int) -> Tuple[Tensor, Tensor]:
    """-> (per-row loss fp32, per-row log-sum-exp fp32); logits [rows, V]."""
    if logits.is_cuda:
        return kx.ce_fwd(logits.contiguous(), target, ignore_index)
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    return F.cross_entropy(lf, target, reduction="none", ignore_index=ignore_index), lse


@ce_fwd.register_fake
def _(logits, target, ignore_index):
    r = logits.new_empty(logits.shape[0], dtype=torch.float32)
    return r, torch.empty_like(r)


@torch.library.custom_op("pfeife::ce_bwd", mutates_args=())
def ce_bwd(dloss: Tensor, logits: Tensor, target: Tensor, lse: Tensor, ignore_index: int) -> Tensor:
    if logits.is_cuda:
        return kx.ce_bwd(logits.contiguous(), target, lse, dloss.float().contiguous(), ignore_index)
    p = torch.exp(logits.float() - lse[:, None])
    valid = target != ignore_index
    onehot = torch.zeros_like(p)
    onehot[valid, target[valid]] = 1.0
    return ((p - onehot) * (dloss.float() * valid)[:, None]).to(logits.dtype)


@ce_bwd.register_fake
def _(dloss, logits, target, lse, ignore_index):
    return torch.empty_like(logits)


def _ce_setup(ctx, inputs, output):
    logits, target, ignore_index = inputs
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(logits, target, output[1])
    ctx.ignore_index = ignore_index


ce_fwd.register_autograd(
    lambda ctx, dloss, dlse: ((None if dloss is None else
                               ce_bwd(dloss.contiguous(), ctx.saved_tensors[0],
                                      ctx.saved_tensors[1], ctx.saved_tensors[2],
                                      ctx.ignore_index)), None, None),
    setup_context=_ce_setup)


def cross_entropy(logits: Tensor, target: Tensor, ignore_index: int = -100,
                  reduction: str = "mean") -> Tensor:
    """Fused log-softmax + NLL over the last dim; the probabilities are never materialised in
    the forward and the backward is one pass over the logits."""
    V = logits.shape[-1]
    loss, _ = ce_fwd(logits.reshape(-1, V), target.reshape(-1), ignore_index)
    if reduction == "none":
        return loss.view(target.shape)
    if reduction == "sum":
        return loss.sum()
    valid = (target.reshape(-1) != ignore_index).sum().clamp(min=1)
    return loss.sum() / valid


@torch.library.custom_op("pfeife::mse_fwd", mutates_args=())
def mse_fwd(a: Tensor, b: Tensor) -> Tensor:
    if _native(a) or (a.is_cuda and a.dtype == torch.float32):
        return kx.mse_fwd(a, b.to(a.dtype)).view(())
    return F.mse_loss(a.float(), b.float())


@mse_fwd.register_fake
def _(a, b):
    return a.new_empty((), dtype=torch.float32)


@torch.library.custom_op("pfeife::mse_bwd", mutates_args=())
def mse_bwd(g: Tensor, a: Tensor, b: Tensor) -> Tensor:
    if _native(a) or (a.is_cuda and a.dtype == torch.float32):
        return kx.mse_bwd(a, b.to(a.dtype), g.reshape(1)).view(a.shape)
    return (2.0 * (a.float() - b.float()) * g.float() / a.numel()).to(a.dtype)


@mse_bwd.register_fake
def _(g, a, b):
    return torch.empty_like(a)


mse_fwd.register_autograd(
    lambda ctx, g: (mse_bwd(g, *ctx.saved_tensors), None),
    setup_context=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0], inputs[1]))


def mse_loss(a: Tensor, b: Tensor) -> Tensor:
    return mse_fwd(a, b)


# =========================================================================== embedding / rope
@torch.library.custom_op("pfeife::embed_fwd", mutates_args=())
def embed_fwd(ids: Tensor, table: Tensor, out_dtype: torch.dtype) -> Tensor:
    if table.is_cuda:
        t = table
        s = _slot(table)
        if s is not None and s.lp is not None and s.lp.dtype == out_dtype:
            t = _weight_as(table, out_dtype)     # the 16-bit shadow: half the bytes, same values
        elif t.dtype != out_dtype and t.dtype != torch.float32:
            t = t.float()
        return kx.embed_fwd(t, ids, out_dtype)
    return F.embedding(ids, table).to(out_dtype)


@embed_fwd.register_fake
def _(ids, table, out_dtype):
    return table.new_empty(ids.shape + (table.shape[1],), dtype=out_dtype)


@torch.library.custom_op("pfeife::embed_bwd", mutates_args=())
def embed_bwd(dout: Tensor, ids: Tensor, table: Tensor) -> Tensor:
    """-> fp32 gradient table (empty when it was accumulated into a registered bucket)."""
    slot = _slot(table)
    if table.is_cuda:
        if slot is not None and slot.main_grad is not None:
            kx.embed_bwd(dout, ids, slot.main_grad.view(table.shape))
            return dout.new_empty(0, dtype=torch.float32)
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        return kx.embed_bwd(dout, ids, g)
    g = torch.zeros(table.shape, dtype=torch.float32)
    return g.index_add_(0, ids.reshape(-1), dout.reshape(-1, table.shape[1]).float())


@embed_bwd.register_fake
def _(dout, ids, table):
    return table.new_empty(table.shape, dtype=torch.float32)


def _embed_backward(ctx, dout):
    ids, table = ctx.saved_tensors
    g = embed_bwd(dout.contiguous(), ids, table)
    return None, (g.to(table.dtype) if g.numel() else None), None


embed_fwd.register_autograd(
    _embed_backward,
    setup_context=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0], inputs[1]))


def embedding(ids: Tensor, table: Tensor, out_dtype: Optional[torch.dtype] = None) -> Tensor:
    if out_dtype is None:
        out_dtype = compute_dtype(table)
    return embed_fwd(ids, table, out_dtype)


@torch.library.custom_op("pfeife::rope_apply", mutates_args=())
def rope_apply(x: Tensor, cos: Tensor, sin: Tensor, inverse: bool) -> Tensor:
    """x [B, S, H, D]; cos/sin fp32 [S, D/2]; half-split pairing (i, i + D/2)."""
    if _native(x) or (x.is_cuda and x.dtype == torch.float32):
        return kx.rope(x if x.stride(-1) == 1 else x.contiguous(), cos.float(), sin.float(), inverse)
    D = x.shape[-1]
    xf = x.float()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    c = cos.float()[None, :, None, :]
    s = sin.float()[None, :, None, :]
    if inverse:
        s = -s
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


@rope_apply.register_fake
def _(x, cos, sin, inverse):
    return torch.empty_like(x)


def _rope_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[1], inputs[2])
    ctx.inverse = inputs[3]


rope_apply.register_autograd(
    lambda ctx, dy: (rope_apply(dy.contiguous(), ctx.saved_tensors[0], ctx.saved_tensors[1],
                                not ctx.inverse), None, None, None),
    setup_context=_rope_setup)


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    return rope_apply(x, cos, sin, False)


def rope_tables(seq_len: int, head_dim: int, theta: float = 10000.0, device=None
                ) -> Tuple[Tensor, Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32)
                           / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


# =========================================================================== attention
def _sdpa_ref(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float
              ) -> Tuple[Tensor, Tensor]:
    """fp32 reference: q,k,v [B, S, H, D] -> (o [B, Sq, H, D], lse [B, H, Sq])."""
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


@torch.library.custom_op("pfeife::attn_fwd", mutates_args=())
def attn_fwd(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float) -> Tuple[Tensor, Tensor]:
    """Flash attention forward.  q [B, Sq, H, D], k/v [B, Sk, H, D] (any strides with a unit
    inner stride) -> (o [B, Sq, H, D] contiguous, lse fp32 [B, H, Sq])."""
    if _native(q) and kx.attention_supported(q, k, v):
        return kx.attn_fwd(q, k, v, causal, scale)
    o, lse = _sdpa_ref(q, k, v, causal, scale)
    return o.contiguous(), lse.contiguous()


@attn_fwd.register_fake
def _(q, k, v, causal, scale):
    B, Sq, H, D = q.shape
    return q.new_empty((B, Sq, H, D)), q.new_empty((B, H, Sq), dtype=torch.float32)


@torch.library.custom_op("pfeife::attn_bwd", mutates_args=())
def attn_bwd(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, causal: bool,
             scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    if _native(q) and kx.attention_supported(q, k, v):
        return kx.attn_bwd(do, q, k, v, o, lse, causal, scale)
    qf, kf, vf, dof = (t.float().permute(0, 2, 1, 3) for t in (q, k, v, do))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse[..., None])
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * o.float().permute(0, 2, 1, 3)).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    back = lambda t, like: t.permute(0, 2, 1, 3).to(like.dtype).contiguous()
    return back(dq, q), back(dk, k), back(dv, v)


@attn_bwd.register_fake
def _(do, q, k, v, o, lse, causal, scale):
    return (q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape))


def _attn_setup(ctx, inputs, output):
    q, k, v, causal, scale = inputs
    o, lse = output
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.causal, ctx.scale = causal, scale


def _attn_backward(ctx, do, dlse):
    q, k, v, o, lse = ctx.saved_tensors
    if do is None:
        return (None,) * 5
    dq, dk, dv = attn_bwd(do.contiguous(), q, k, v, o, lse, ctx.causal, ctx.scale)
    return dq, dk, dv, None, None


attn_fwd.register_autograd(_attn_backward, setup_context=_attn_setup)


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = False,
              scale: Optional[float] = None) -> Tensor:
    """softmax(q k^T * scale [+ causal mask]) v without materialising the score matrix.
    Layout [batch, seq, heads, head_dim]; q/k/v may be strided views of a fused projection."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return attn_fwd(q, k, v, causal, float(scale))[0]


# --------------------------------------------------------------------------- packed self-attention
@torch.library.custom_op("pfeife::attn_qkv_fwd", mutates_args=())
def attn_qkv_fwd(qkv: Tensor, causal: bool, scale: float) -> Tuple[Tensor, Tensor]:
    """Self-attention on a fused projection qkv [B, S, 3, H, D] -> (o [B, S, H, D], lse)."""
    return attn_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal, scale)


@attn_qkv_fwd.register_fake
def _(qkv, causal, scale):
    B, S, _, H, D = qkv.shape
    return qkv.new_empty((B, S, H, D)), qkv.new_empty((B, H, S), dtype=torch.float32)


@torch.library.custom_op("pfeife::attn_qkv_bwd", mutates_args=())
def attn_qkv_bwd(do: Tensor, qkv: Tensor, o: Tensor, lse: Tensor, causal: bool,
                 scale: float) -> Tensor:
    """-> d(qkv) [B, S, 3, H, D], written in place by the backward kernels (no concatenation)."""
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    if _native(qkv) and kx.attention_supported(q, k, v):
        dq, _, _ = kx.attn_bwd(do, q, k, v, o, lse, causal, scale, packed=True)
        return dq._base if dq._base is not None else torch.stack(
            kx.attn_bwd(do, q, k, v, o, lse, causal, scale), dim=2)
    dq, dk, dv = attn_bwd(do, q, k, v, o, lse, causal, scale)
    return torch.stack([dq, dk, dv], dim=2)


@attn_qkv_bwd.register_fake
def _(do, qkv, o, lse, causal, scale):
    return torch.empty_like(qkv)


def _attn_qkv_setup(ctx, inputs, output):
    qkv, causal, scale = inputs
    o, lse = output
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(qkv, o, lse)
    ctx.causal, ctx.scale = causal, scale


def _attn_qkv_backward(ctx, do, dlse):
    qkv, o, lse = ctx.saved_tensors
    if do is None:
        return None, None, None
    return attn_qkv_bwd(do.contiguous(), qkv, o, lse, ctx.causal, ctx.scale), None, None


attn_qkv_fwd.register_autograd(_attn_qkv_backward, setup_context=_attn_qkv_setup)


def attention_qkv(qkv: Tensor, causal: bool = False, scale: Optional[float] = None) -> Tensor:
    """Self-attention directly on a fused QKV projection laid out [B, S, 3, H, D]."""
    if scale is None:
        scale = 1.0 / math.sqrt(qkv.shape[-1])
    return attn_qkv_fwd(qkv, causal, float(scale))[0]


# =========================================================================== UNet ops (NHWC)
def _pad_to8(n: int) -> int:
    return (n + 7) // 8 * 8


@torch.library.custom_op("pfeife::conv2d_fwd", mutates_args=())
def conv2d_fwd(x: Tensor, w: Tensor, bias: Optional[Tensor], stride: int, pad: int) -> Tensor:
    """Channels-last convolution: x [B, H, W, Cin], w [Cout, Cin, KH, KW] -> [B, Ho, Wo, Cout].
    On the native path the convolution is a tcgen05 implicit GEMM (patches read straight from
    x by TMA) when the shape allows it, else a GEMM over im2col rows (1x1: no im2col)."""
    Cout, Cin, KH, KW = w.shape
    cd = compute_dtype(x)
    if x.is_cuda and cd in (torch.float16, torch.bfloat16):
        xc = x if x.dtype == cd else kx.cast(x, cd)
        B, H, W, _ = xc.shape
        cin8, cout8 = _pad_to8(Cin), _pad_to8(Cout)
        if cin8 != Cin:
            xc = F.pad(xc, (0, cin8 - Cin))
        w2 = _weight_as(w, cd).permute(0, 2, 3, 1)                      # [Cout, KH, KW, Cin]
        if cin8 != Cin or cout8 != Cout:
            w2 = F.pad(w2, (0, cin8 - Cin, 0, 0, 0, 0, 0, cout8 - Cout))
        w2 = w2.reshape(cout8, KH * KW * cin8).contiguous()
        Ho = (H + 2 * pad - KH) // stride + 1
        Wo = (W + 2 * pad - KW) // stride + 1
        b2 = None
        if bias is not None:
            b2 = bias.float() if cout8 == Cout else F.pad(bias.float(), (0, cout8 - Cout))
        one = KH == 1 and KW == 1 and stride == 1 and pad == 0
        if not one and cin8 == Cin and kx.conv_gemm_supported(xc.contiguous(), KH, KW, stride, pad):
            y = kx.conv_gemm(xc.contiguous(), w2, KH, KW, stride, pad, bias=b2)
            return y[..., :Cout].contiguous() if cout8 != Cout else y
        cols = xc.reshape(B * H * W, cin8) if one else kx.im2col(xc, KH, KW, stride, pad)
        y = kx.gemm(cols, w2, bias=b2)
        y = y.view(B, Ho, Wo, cout8)
        return y[..., :Cout].contiguous() if cout8 != Cout else y
    y = F.conv2d(x.to(cd).permute(0, 3, 1, 2), w.to(cd), None if bias is None else bias.to(cd),
                 stride=stride, padding=pad)
    return y.permute(0, 2, 3, 1).contiguous()


@conv2d_fwd.register_fake
def _(x, w, bias, stride, pad):
    B, H, W, _ = x.shape
    Cout, _, KH, KW = w.shape
    Ho = (H + 2 * pad - KH) // stride + 1
    Wo = (W + 2 * pad - KW) // stride + 1
    return x.new_empty((B, Ho, Wo, Cout), dtype=compute_dtype(x))


@torch.library.custom_op("pfeife::conv2d_bwd", mutates_args=())
def conv2d_bwd(dy: Tensor, x: Tensor, w: Tensor, stride: int, pad: int, need_dx: bool,
               need_db: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """-> (dx [B,H,W,Cin], dw fp32 [Cout,Cin,KH,KW], db fp32 [Cout])."""
    Cout, Cin, KH, KW = w.shape
    cd = dy.dtype
    if dy.is_cuda and cd in (torch.float16, torch.bfloat16):
        xc = x if x.dtype == cd else kx.cast(x, cd)
        B, H, W, _ = xc.shape
        cin8, cout8 = _pad_to8(Cin), _pad_to8(Cout)
        if cin8 != Cin:
            xc = F.pad(xc, (0, cin8 - Cin))
        dy2 = dy.reshape(-1, Cout)
        if cout8 != Cout:
            dy2 = F.pad(dy2, (0, cout8 - Cout))
        dy2 = dy2.contiguous()
        one = KH == 1 and KW == 1 and stride == 1 and pad == 0
        if not one and cin8 == Cin and \
                kx.conv_wgrad_supported(xc.contiguous(), cout8, KH, KW, stride, pad):
            dw2 = kx.conv_wgrad(dy2, xc.contiguous(), KH, KW, stride, pad)       # [cout8, K]
        else:
            cols = xc.reshape(B * H * W, cin8) if one else kx.im2col(xc, KH, KW, stride, pad)
            dw2 = kx.gemm(dy2, cols, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dw = dw2.view(cout8, KH, KW, cin8)[:Cout, :, :, :Cin].permute(0, 3, 1, 2).contiguous()
        dx = dy.new_empty(0)
        if need_dx:
            w2 = _weight_as(w, cd).permute(0, 2, 3, 1)
            if cin8 != Cin or cout8 != Cout:
                w2 = F.pad(w2, (0, cin8 - Cin, 0, 0, 0, 0, 0, cout8 - Cout))
            w2 = w2.reshape(cout8, KH * KW * cin8).contiguous()
            dy4 = dy2.view(B, -1, dy.shape[2], cout8)
            if not one and stride == 1 and cout8 == Cout and \
                    kx.conv_gemm_supported(dy4, KH, KW, 1, KH - 1 - pad) and \
                    dy4.shape[1] + 2 * (KH - 1 - pad) - KH + 1 == H:
                # dx = correlation of dy with the taps flipped and the channel roles swapped
                wt = _weight_as(w, cd).flip(2, 3).permute(1, 2, 3, 0)     # [Cin, KH, KW, Cout]
                if cin8 != Cin:
                    wt = F.pad(wt, (0, 0, 0, 0, 0, 0, 0, cin8 - Cin))
                wt = wt.reshape(cin8, KH * KW * cout8).contiguous()
                dxp = kx.conv_gemm(dy4, wt, KH, KW, 1, KH - 1 - pad)
            else:
                dcols = kx.gemm(dy2, w2, b_mn=True)                              # [M, K]
                dxp = dcols.view(B, H, W, cin8) if one else \
                    kx.col2im(dcols, (B, H, W, cin8), KH, KW, stride, pad)
            dx = dxp[..., :Cin].contiguous() if cin8 != Cin else dxp
        db = kx.colsum(dy2)[:Cout].contiguous() if need_db else dy.new_empty(0, dtype=torch.float32)
        return dx, dw, db
    xn = x.to(cd).permute(0, 3, 1, 2)
    dyn = dy.permute(0, 3, 1, 2)
    dx = torch.nn.grad.conv2d_input(xn.shape, w.to(cd), dyn, stride=stride, padding=pad) \
        .permute(0, 2, 3, 1).contiguous() if need_dx else dy.new_empty(0)
    dw = torch.nn.grad.conv2d_weight(xn.float(), w.shape, dyn.float(), stride=stride, padding=pad)
    db = dyn.float().sum((0, 2, 3)) if need_db else dy.new_empty(0, dtype=torch.float32)
    return dx, dw.float(), db


@conv2d_bwd.register_fake
def _(dy, x, w, stride, pad, need_dx, need_db):
    return (torch.empty_like(x, dtype=dy.dtype) if need_dx else dy.new_empty(0),
            w.new_empty(w.shape, dtype=torch.float32),
            dy.new_empty(w.shape[0] if need_db else 0, dtype=torch.float32))


def _conv_setup(ctx, inputs, output):
    x, w, bias, stride, pad = inputs
    ctx.save_for_backward(x, w)
    ctx.stride, ctx.pad = stride, pad
    ctx.meta = (x.dtype, w.dtype, None if bias is None else bias.dtype)


def _conv_backward(ctx, dy):
    x, w = ctx.saved_tensors
    xd, wd, bd = ctx.meta
    need = ctx.needs_input_grad
    dx, dw, db = conv2d_bwd(dy.contiguous(), x, w, ctx.stride, ctx.pad, need[0], bd is not None)
    return (dx.to(xd) if need[0] else None, dw.to(wd) if need[1] else None,
            db.to(bd) if bd is not None else None, None, None)


conv2d_fwd.register_autograd(_conv_backward, setup_context=_conv_setup)


def conv2d(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, stride: int = 1,
           padding: int = 0) -> Tensor:
    """NHWC convolution with a standard [Cout, Cin, KH, KW] weight."""
    return conv2d_fwd(x, weight, bias, stride, padding)


@torch.library.custom_op("pfeife::group_norm_fwd", mutates_args=())
def group_norm_fwd(x: Tensor, gamma: Tensor, beta: Tensor, groups: int, eps: float,
                   silu_act: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """NHWC GroupNorm with optional fused SiLU -> (y, mean[B*G], rstd[B*G])."""
    if _native(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return kx.groupnorm_fwd(x, gamma, beta, groups, eps, silu_act)
    B, H, W, C = x.shape
    xf = x.float().reshape(B, H * W, groups, C // groups)
    mean = xf.mean((1, 3))
    var = xf.var((1, 3), unbiased=False)
    rstd = torch.rsqrt(var + eps)
    xh = (xf - mean[:, None, :, None]) * rstd[:, None, :, None]
    y = xh.reshape(B, H, W, C) * gamma.float() + beta.float()
    if silu_act:
        y = F.silu(y)
    return y.to(x.dtype), mean.reshape(-1), rstd.reshape(-1)


@group_norm_fwd.register_fake
def _(x, gamma, beta, groups, eps, silu_act):
    s = x.new_empty(x.shape[0] * groups, dtype=torch.float32)
    return torch.empty_like(x), s, torch.empty_like(s)


@torch.library.custom_op("pfeife::group_norm_bwd", mutates_args=())
def group_norm_bwd(dy: Tensor, x: Tensor, mean: Tensor, rstd: Tensor, gamma: Tensor, beta: Tensor,
                   groups: int, silu_act: bool) -> Tuple[Tensor, Tensor, Tensor]:
    if _native(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return kx.groupnorm_bwd(dy, x, mean, rstd, gamma, beta, groups, silu_act)
    B, H, W, C = x.shape
    cpg = C // groups
    xf = x.float().reshape(B, H * W, groups, cpg)
    xh = (xf - mean.view(B, 1, groups, 1)) * rstd.view(B, 1, groups, 1)
    g = gamma.float().view(1, 1, groups, cpg)
    dz = dy.float().reshape(B, H * W, groups, cpg)
    if silu_act:
        z = xh * g + beta.float().view(1, 1, groups, cpg)
        dz = dz * _dact_ref(z, ACT_SILU)
    dgamma = (dz * xh).sum((0, 1)).reshape(C)
    dbeta = dz.sum((0, 1)).reshape(C)
    dzg = dz * g
    n = H * W * cpg
    a = dzg.sum((1, 3), keepdim=True) / n
    b = (dzg * xh).sum((1, 3), keepdim=True) / n
    dx = rstd.view(B, 1, groups, 1) * (dzg - a - xh * b)
    return dx.reshape(B, H, W, C).to(x.dtype), dgamma, dbeta


@group_norm_bwd.register_fake
def _(dy, x, mean, rstd, gamma, beta, groups, silu_act):
    C = x.shape[-1]
    return (torch.empty_like(x), x.new_empty(C, dtype=torch.float32),
            x.new_empty(C, dtype=torch.float32))


def _gn_setup(ctx, inputs, output):
    x, gamma, beta, groups, eps, silu_act = inputs
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(x, output[1], output[2], gamma, beta)
    ctx.groups, ctx.silu_act = groups, silu_act


def _gn_backward(ctx, dy, dmean, drstd):
    x, mean, rstd, gamma, beta = ctx.saved_tensors
    if dy is None:
        return (None,) * 6
    dx, dg, db = group_norm_bwd(dy.contiguous(), x, mean, rstd, gamma, beta, ctx.groups,
                                ctx.silu_act)
    return dx, dg.to(gamma.dtype), db.to(beta.dtype), None, None, None


group_norm_fwd.register_autograd(_gn_backward, setup_context=_gn_setup)


def group_norm(x: Tensor, weight: Tensor, bias: Tensor, groups: int = 32, eps: float = 1e-5,
               silu: bool = False) -> Tensor:
    """GroupNorm over an NHWC tensor, optionally followed by SiLU in the same kernel."""
    return group_norm_fwd(x, weight, bias, groups, eps, silu)[0]


@torch.library.custom_op("pfeife::upsample2x_op", mutates_args=())
def upsample2x_op(x: Tensor, backward: bool) -> Tensor:
    if _native(x) and x.shape[-1] % 8 == 0:
        return kx.upsample2x(x, backward)
    if not backward:
        return x.repeat_interleave(2, 1).repeat_interleave(2, 2)
    B, H2, W2, C = x.shape
    return x.float().reshape(B, H2 // 2, 2, W2 // 2, 2, C).sum((2, 4)).to(x.dtype)


@upsample2x_op.register_fake
def _(x, backward):
    B, H, W, C = x.shape
    return x.new_empty((B, H // 2, W // 2, C) if backward else (B, 2 * H, 2 * W, C))


upsample2x_op.register_autograd(
    lambda ctx, dy: (upsample2x_op(dy.contiguous(), not ctx.backward), None),
    setup_context=lambda ctx, inputs, output: setattr(ctx, "backward", inputs[1]))


def upsample_nearest2x(x: Tensor) -> Tensor:
    return upsample2x_op(x, False)
