"""Per-rank parameter store: flat fp32 master weights, flat fp32 gradient bucket, optimizer
moments and (under mixed precision) a flat 16-bit shadow, with the optimizer step as one fused
kernel per parameter group.

The stage graphs receive *views* of these flat buffers: an fp32 master view whose ``.grad`` is
preset to the matching view of the gradient bucket (so autograd accumulates in place across
micro-batches), registered with the ops layer so that ``linear`` reads the 16-bit shadow and
its wgrad epilogue accumulates straight into the bucket.  The flat layout is what the fused
data-parallel kernel reduces, updates and re-distributes shard by shard.

The user's optimizer object stays the source of hyper-parameters: every step the main rank
snapshots its ``param_groups`` (lr, betas, eps, weight_decay, momentum ...) and the values
travel with the step's control message, so LR schedulers attached to the user's optimizer take
effect on every rank (the reference's worker-side optimizer copies never see LR updates,
pfeife/mp/worker.py:265-275).  Adam, AdamW and SGD run on the native kernels; any other
``torch.optim`` class is instantiated over the master views and stepped as is.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..ops import kernels as kx
from ..option import get_optimizer_cls

ALIGN = 128  # elements; keeps every view 16-byte aligned in fp32 and in 16-bit

_HYPER_KEYS = ("lr", "betas", "eps", "weight_decay", "momentum", "dampening", "nesterov",
               "amsgrad", "maximize")


def gather_deferrable(t: torch.Tensor) -> bool:
    """A weight whose 16-bit copy may stay row-sharded between the optimizer step and its first
    consumer: a matrix a linear layer reads (rows = output features), wide enough for 16-byte
    row transfers and large enough for the transfer to matter."""
    return t.dim() == 2 and t.shape[1] % 8 == 0 and t.shape[0] >= 256 and t.numel() >= (1 << 18)


def snapshot_hyper(optimizer) -> List[Dict[str, Any]]:
    """The picklable hyper-parameters of every param group of a torch optimizer."""
    out = []
    for g in optimizer.param_groups:
        out.append({k: (tuple(v) if isinstance(v, (list, tuple)) else v) for k, v in g.items()
                    if k != "params" and isinstance(v, (int, float, bool, tuple, list, type(None)))})
    return out


@dataclass
class StateEntry:
    ph_index: int
    qualname: str
    kind: str                 # "param" | "buffer"
    tensor: torch.Tensor      # initial value (any device)
    requires_grad: bool
    group: int = 0            # index into the user's optimizer.param_groups
    # True: every op that reads this parameter reads its 16-bit shadow (a weight of linear /
    # conv / embedding); False: some op reads the fp32 value; None: not analysed
    lp_only: Optional[bool] = None


@dataclass
class _Slot:
    entry: StateEntry
    offset: int = -1          # element offset in the flat buffers (-1: not packed)
    numel: int = 0
    view: Optional[torch.Tensor] = None       # what the stage graph is given
    master: Optional[torch.Tensor] = None
    grad: Optional[torch.Tensor] = None
    lp: Optional[torch.Tensor] = None
    deferred: bool = False    # all-gather of `lp` left to its first consumer


class RankParams:
    def __init__(self, entries: Sequence[StateEntry], device: torch.device,
                 lp_dtype: Optional[torch.dtype], optimizer_type: str,
                 hyper: List[Dict[str, Any]], native: Optional[bool] = None,
                 alloc=None, defer_gather: bool = False):
        """`alloc(numel, dtype) -> Tensor` lets the data-parallel layer place the flat buffers
        in peer-accessible memory.  With `defer_gather` the matrices that linear layers consume
        are packed first within their optimizer group, so that the data-parallel step can leave
        the all-gather of their 16-bit copies to the first GEMM that reads them
        (``deferred_below`` = end of that region per group)."""
        self.device = device
        self.lp_dtype = lp_dtype
        self.optimizer_type = optimizer_type.lower()
        self.hyper = [dict(h) for h in hyper] or [{}]
        self.native = (device.type == "cuda") if native is None else native
        if any(h.get("amsgrad") or h.get("maximize") for h in self.hyper):
            self.native = False      # variants the native kernels do not implement
        self.step_count = 0
        # optimizer steps that were applied (not skipped on an overflow): drives Adam's bias
        # correction on the device
        self.applied_steps = torch.zeros(1, dtype=torch.int32, device=device) \
            if device.type == "cuda" else None
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))

        packed = [e for e in entries if e.kind == "param" and e.requires_grad
                  and e.tensor.dtype.is_floating_point]
        defer = bool(defer_gather and lp_dtype is not None and self.native)
        deferrable = (lambda e: defer and gather_deferrable(e.tensor) and e.lp_only is not False)
        # Within a group: first the matrices whose all-gather is deferred, then the other weights
        # that are only read through their shadow, then what some op reads in fp32.  The fused
        # data-parallel step pushes fp32 masters to the replicas only from `master_from` on; a
        # group with a parameter that was not analysed is pushed as a whole.
        shadow_only = (lambda e: e.lp_only is True and lp_dtype is not None)
        packed.sort(key=lambda e: (e.group, not deferrable(e), not shadow_only(e), e.ph_index))
        self.slots: Dict[int, _Slot] = {}
        self.group_ranges: List[Tuple[int, int, int]] = []   # (group, lo, hi)
        self.deferred_below: Dict[int, int] = {}             # group -> end of its deferred region
        self.master_from: Dict[int, int] = {}                # group -> start of its fp32-read tail
        unknown = {e.group for e in packed if e.lp_only is None}
        off = 0
        cur_group, group_lo = None, 0
        for e in packed:
            if e.group != cur_group:
                if cur_group is not None:
                    self.group_ranges.append((cur_group, group_lo, off))
                cur_group, group_lo = e.group, off
                self.deferred_below[e.group] = off
                self.master_from[e.group] = off
            n = e.tensor.numel()
            self.slots[e.ph_index] = _Slot(e, off, n, deferred=deferrable(e))
            off += (n + ALIGN - 1) // ALIGN * ALIGN
            if deferrable(e):
                self.deferred_below[e.group] = off
            if shadow_only(e) and e.group not in unknown:
                self.master_from[e.group] = off
        if cur_group is not None:
            self.group_ranges.append((cur_group, group_lo, off))
        self.numel = off
        self.master = alloc(off, torch.float32)
        self.grad = alloc(off, torch.float32)
        self.lp = alloc(off, lp_dtype) if (lp_dtype is not None and off) else None
        self.opt_state: Dict[str, torch.Tensor] = {}
        self.found_inf = torch.zeros(1, dtype=torch.float32, device=device)
        self._torch_opt = None
        self._pending_opt_state = None
        self.dp_state = None     # fused data-parallel layer that owns sharded optimizer moments

        with torch.no_grad():
            for s in self.slots.values():
                e = s.entry
                s.master = self.master[s.offset:s.offset + s.numel].view(e.tensor.shape)
                s.master.copy_(e.tensor.detach().to(device=device, dtype=torch.float32))
                s.grad = self.grad[s.offset:s.offset + s.numel].view(e.tensor.shape)
                if self.lp is not None:
                    s.lp = self.lp[s.offset:s.offset + s.numel].view(e.tensor.shape)
                    s.lp.copy_(s.master)
                if e.tensor.dtype == torch.float32 or self.lp is None or \
                        e.tensor.dtype != self.lp.dtype:
                    v = s.master.detach()
                    v.requires_grad_(True)
                    v.grad = s.grad
                else:   # the model itself is 16-bit: bind the shadow, fold its grads by hook
                    v = s.lp.detach()
                    v.requires_grad_(True)
                    v.register_post_accumulate_grad_hook(self._fold_lp_grad(s))
                s.view = v
                ops.register_param(s.master, s.lp, s.grad if self.native else None)
        for e in entries:
            if e.ph_index in self.slots:
                continue
            t = e.tensor.detach().to(device)
            if e.kind == "param" and e.requires_grad and not t.dtype.is_floating_point:
                t = t.clone()
            self.slots[e.ph_index] = _Slot(e, -1, t.numel(), view=t)

    def _fold_lp_grad(self, s: _Slot):
        def hook(p: torch.Tensor):
            if p.grad is not None:
                s.grad.add_(p.grad.to(torch.float32))
                p.grad = None
        return hook

    # ------------------------------------------------------------------ access
    def tensor_for(self, ph_index: int) -> torch.Tensor:
        return self.slots[ph_index].view

    def packed_slots(self) -> List[_Slot]:
        return [s for s in self.slots.values() if s.offset >= 0]

    def prepare_backward(self) -> None:
        """(Re)attaches the bucket views as ``.grad`` so autograd accumulates in place."""
        for s in self.packed_slots():
            if s.view.dtype == torch.float32 and s.view.grad is not s.grad:
                s.view.grad = s.grad

    def zero_grad(self) -> None:
        if self.numel:
            self.grad.zero_()

    def set_hyper(self, hyper: Optional[List[Dict[str, Any]]]) -> None:
        if hyper:
            self.hyper = [dict(h) for h in hyper]

    # ------------------------------------------------------------------ optimizer
    def _state(self, name: str) -> torch.Tensor:
        if name not in self.opt_state:
            self.opt_state[name] = torch.zeros(self.numel, dtype=torch.float32,
                                               device=self.device)
        return self.opt_state[name]

    def check_finite(self) -> None:
        """Sets ``found_inf`` when any accumulated gradient is non-finite."""
        if not self.numel:
            return
        if self.native:
            kx.nonfinite(self.grad, self.found_inf)
        else:
            self.found_inf.fill_(0.0 if bool(torch.isfinite(self.grad).all()) else 1.0)

    def step(self, grad_scale: float = 1.0, loss_scale: Optional[torch.Tensor] = None,
             use_found_inf: bool = False, shard: Optional[Tuple[int, int]] = None) -> None:
        """One optimizer step on [lo, hi) of every group (the whole range by default), then
        zeroes the gradient it consumed.  Skipped on the device when ``found_inf`` is set."""
        self.step_count += 1
        if not self.numel:
            return
        kind = self.optimizer_type
        if kind in ("adam", "adamw", "sgd") and self.native:
            self._step_native(kind, grad_scale, loss_scale, use_found_inf, shard)
        else:
            self._step_torch(grad_scale, loss_scale, use_found_inf)

    def _ranges(self, shard):
        for g, lo, hi in self.group_ranges:
            if shard is not None:
                lo, hi = max(lo, shard[0]), min(hi, shard[1])
            if hi > lo:
                yield g, lo, hi

    def _step_native(self, kind, grad_scale, loss_scale, use_found_inf, shard) -> None:
        found = self.found_inf if use_found_inf else None
        self._step_groups(kind, grad_scale, loss_scale, found, shard)
        if kind in ("adam", "adamw"):
            kx.step_advance(self.applied_steps, found)

    def _step_groups(self, kind, grad_scale, loss_scale, found, shard) -> None:
        for g, lo, hi in self._ranges(shard):
            h = self.hyper[min(g, len(self.hyper) - 1)]
            p, gr = self.master[lo:hi], self.grad[lo:hi]
            lp = self.lp[lo:hi] if self.lp is not None else None
            if kind in ("adam", "adamw"):
                b1, b2 = h.get("betas", (0.9, 0.999))
                kx.adamw(p, gr, self._state("exp_avg")[lo:hi], self._state("exp_avg_sq")[lo:hi],
                         lr=h.get("lr", 1e-3), beta1=b1, beta2=b2, eps=h.get("eps", 1e-8),
                         weight_decay=h.get("weight_decay", 0.01 if kind == "adamw" else 0.0),
                         step=self.step_count, grad_scale=grad_scale,
                         decoupled=(kind == "adamw"), zero_grad=True, lp=lp, found_inf=found,
                         loss_scale=loss_scale, applied_steps=self.applied_steps)
            else:
                mom = h.get("momentum", 0.0)
                kx.sgd(p, gr, self._state("momentum")[lo:hi] if mom else None,
                       lr=h.get("lr", 1e-3), momentum=mom, dampening=h.get("dampening", 0.0),
                       weight_decay=h.get("weight_decay", 0.0),
                       nesterov=bool(h.get("nesterov", False)),
                       first_step=(self.step_count == 1), grad_scale=grad_scale, zero_grad=True,
                       lp=lp, found_inf=found, loss_scale=loss_scale)

    def _step_torch(self, grad_scale, loss_scale, use_found_inf) -> None:
        """Reference path: a torch optimizer over the master views (CPU runs and optimizer
        classes without a native kernel)."""
        if self._torch_opt is None:
            groups: Dict[int, List[torch.Tensor]] = {}
            for s in self.packed_slots():
                p = s.master.detach().requires_grad_(True)
                p.grad = s.grad
                s._opt_param = p
                groups.setdefault(s.entry.group, []).append(p)
            cls = get_optimizer_cls(self.optimizer_type)
            pg = []
            # this rank may hold only some of the user's groups: remember which
            self._torch_group_ids = sorted(groups)
            for g in sorted(groups):
                h = {k: v for k, v in self.hyper[min(g, len(self.hyper) - 1)].items()
                     if k in _HYPER_KEYS or k in ("foreach", "fused", "capturable",
                                                  "differentiable")}
                pg.append({"params": groups[g], **h})
            self._torch_opt = cls(pg)
            if self._pending_opt_state is not None:     # a checkpoint loaded before the first step
                self._apply_torch_state(self._pending_opt_state)
                self._pending_opt_state = None
        for i, g in enumerate(self._torch_opt.param_groups):
            h = self.hyper[min(self._torch_group_ids[i], len(self.hyper) - 1)]
            for k in _HYPER_KEYS:
                if k in h and k in g:
                    g[k] = h[k]
        skip = use_found_inf and float(self.found_inf) != 0.0
        if not skip:
            scale = grad_scale
            if loss_scale is not None:
                scale = scale / float(loss_scale.reshape(-1)[0])
            if scale != 1.0:
                self.grad.mul_(scale)
            for s in self.packed_slots():
                s._opt_param.grad = s.grad
            self._torch_opt.step()
            if self.lp is not None:
                self.lp.copy_(self.master)
        self.grad.zero_()

    # ------------------------------------------------------------------ checkpoint
    def named_tensors(self) -> Dict[str, torch.Tensor]:
        """qualified name -> current full-precision value (for gather_params / state_dict)."""
        if self.dp_state is not None and getattr(self.dp_state, "fused", False):
            self.dp_state.gather_master()    # a collective: all replicas checkpoint together
        out = {}
        for s in self.slots.values():
            out[s.entry.qualname] = (s.master if s.offset >= 0 else s.view).detach()
        return out

    def optimizer_steps(self) -> int:
        """Steps that count for Adam's bias correction: on the native path the device counter
        (skipped steps excluded), else the host's count."""
        if self.applied_steps is not None and self.native and \
                self.optimizer_type in ("adam", "adamw"):
            return int(self.applied_steps.item())
        return self.step_count

    def _set_optimizer_steps(self, n: int) -> None:
        self.step_count = int(n)
        if self.applied_steps is not None:
            self.applied_steps.fill_(int(n))

    def optimizer_state(self) -> Dict[str, Dict[str, torch.Tensor]]:
        """qualified name -> {state name -> tensor}, keyed like torch's per-parameter state."""
        out: Dict[str, Dict[str, torch.Tensor]] = {}
        # fused data parallelism keeps each moment only on the rank that owns the shard: assemble
        # full-length copies (a collective over the replicas, which all take checkpoints together)
        flats = self.dp_state.gather_optimizer_state() \
            if (self.dp_state is not None and getattr(self.dp_state, "fused", False)) else None
        steps = self.optimizer_steps()
        for s in self.packed_slots():
            if flats is not None:
                st = {k: v[s.offset:s.offset + s.numel].view(s.entry.tensor.shape).detach().clone()
                      for k, v in flats.items()}
            elif self._torch_opt is not None:
                # reference path: the torch optimizer owns the per-parameter state
                src = self._torch_opt.state.get(getattr(s, "_opt_param", None), {})
                st = {k: v.detach().clone().view(s.entry.tensor.shape)
                      for k, v in src.items() if torch.is_tensor(v) and v.numel() == s.numel
                      and k != "step"}
                if "step" in src:
                    # the optimizer's own count: steps skipped on an overflow are not in it
                    st["step"] = torch.tensor(float(src["step"]))
                    out[s.entry.qualname] = st
                    continue
            else:
                st = {k: v[s.offset:s.offset + s.numel].view(s.entry.tensor.shape).detach().clone()
                      for k, v in self.opt_state.items()}
            st["step"] = torch.tensor(float(steps))
            out[s.entry.qualname] = st
        return out

    def _uses_torch_optimizer(self) -> bool:
        return not (self.optimizer_type in ("adam", "adamw", "sgd") and self.native)

    def _apply_torch_state(self, state: Dict[str, Dict[str, torch.Tensor]]) -> None:
        for s in self.packed_slots():
            st = state.get(s.entry.qualname)
            p = getattr(s, "_opt_param", None)
            if not st or p is None:
                continue
            dst = self._torch_opt.state[p]
            for k, v in st.items():
                if k == "step":
                    continue
                dst[k] = v.detach().to(device=p.device, dtype=p.dtype).reshape(p.shape).clone()
            if "exp_avg" in st:     # Adam family: its own step counter drives the bias correction
                dst["step"] = torch.tensor(float(st.get("step", self.step_count)))

    def load_optimizer_state(self, state: Dict[str, Dict[str, torch.Tensor]]) -> None:
        if self.dp_state is not None and getattr(self.dp_state, "fused", False):
            flats: Dict[str, torch.Tensor] = {}
            for s in self.packed_slots():
                st = state.get(s.entry.qualname)
                if not st:
                    continue
                for k, v in st.items():
                    if k == "step":
                        self._set_optimizer_steps(int(float(v)))
                        continue
                    if k not in flats:
                        flats[k] = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
                    flats[k][s.offset:s.offset + s.numel].copy_(v.reshape(-1))
            self.dp_state.load_optimizer_state(flats)
            return
        if self._uses_torch_optimizer():
            for st in state.values():
                if st and "step" in st:
                    self.step_count = int(float(st["step"]))
                    break
            if self._torch_opt is not None:
                self._apply_torch_state(state)
            else:
                self._pending_opt_state = state
            return
        for s in self.packed_slots():
            st = state.get(s.entry.qualname)
            if not st:
                continue
            for k, v in st.items():
                if k == "step":
                    self._set_optimizer_steps(int(float(v)))
                    continue
                self._state(k)[s.offset:s.offset + s.numel].copy_(v.reshape(-1))

    def load_named(self, tensors: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for s in self.slots.values():
                t = tensors.get(s.entry.qualname)
                if t is None:
                    continue
                if s.offset >= 0:
                    s.master.copy_(t)
                    if s.lp is not None:
                        s.lp.copy_(s.master)
                else:
                    s.view.copy_(t)


class LossScaler:
    """One dynamic loss scale for the whole job (the reference keeps one GradScaler per worker
    plus the user's own, so scales compound stage by stage, pfeife/mp/worker.py:133-145 and
    :1580-1587).  The scale and its growth tracker live on the device; the update after each
    step is one tiny kernel, and the skip decision is read by the optimizer kernel itself."""

    def __init__(self, device: torch.device, enabled: bool, init_scale: float = 65536.0,
                 growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000):
        self.enabled = enabled
        self.device = device
        self.growth, self.backoff, self.interval = growth_factor, backoff_factor, growth_interval
        self.state = torch.tensor([init_scale if enabled else 1.0, 0.0], dtype=torch.float32,
                                  device=device)

    @property
    def scale_tensor(self) -> Optional[torch.Tensor]:
        return self.state[:1] if self.enabled else None

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        if not self.enabled:
            return loss
        return loss * self.state[0].to(loss.dtype)

    def get_scale(self) -> float:
        return float(self.state[0])

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """Scale and growth tracker, for checkpoints: a resumed fp16 run continues at the scale
        the job had settled on instead of overflowing its way down from the initial one."""
        st = self.state.detach().cpu()
        return {"scale": st[0].clone(), "growth_tracker": st[1].clone()}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        if not self.enabled or not sd:
            return
        self.state[0] = float(sd["scale"])
        self.state[1] = float(sd.get("growth_tracker", 0.0))

    def update(self, found_inf: torch.Tensor) -> None:
        if not self.enabled:
            return
        if self.device.type == "cuda":
            kx.loss_scale_update(self.state, found_inf, self.growth, self.backoff, self.interval)
        else:
            if float(found_inf) != 0.0:
                self.state[0] *= self.backoff
                self.state[1] = 0.0
            else:
                self.state[1] += 1
                if int(self.state[1]) >= self.interval:
                    self.state[0] *= self.growth
                    self.state[1] = 0.0
            found_inf.zero_()
