"""Flat-buffer AdamW (kernel K11) with an optional fp32 master copy.

All trainable parameters of a model are re-pointed into ONE contiguous buffer (and
their ``.grad`` into one contiguous gradient buffer), so the optimiser step, the
global gradient norm and any gradient collective are each a single launch over a
flat array instead of one per tensor.  The update is decoupled-weight-decay Adam:

    g   = grad * clip_coef                      (clip_coef stays on the device)
    m   = b1 m + (1-b1) g ;  v = b2 v + (1-b2) g^2
    w  -= lr * ( (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps) + wd * w )

computed on the fp32 master weights and re-cast to the parameter dtype in the same
pass.  ``state_dict()`` uses the ``torch.optim.AdamW`` layout (state keyed by
parameter index with ``step`` / ``exp_avg`` / ``exp_avg_sq``) so checkpoints stay
interchangeable (reference optimiser: ``vrl/trainers/online.py:33-56,322-341``); for
low-precision parameters each entry additionally carries the fp32 ``master`` copy
(a key ``torch.optim.AdamW`` ignores), so a resumed run continues from exactly the
weights the interrupted run held rather than from their bf16 rounding.

Parameters that a :class:`visionrl_b200.parallel.fsdp.ShardedParamRuntime` has sharded
(marked ``_vrl_sharded``) are not flattened here — the runtime owns their shards,
moments and update — but they keep their place in ``state_dict()``: their state is
gathered to the full ``[N, K]`` shape on save and sliced on load, so a checkpoint
does not depend on the number of ranks that wrote it.
"""

from __future__ import annotations

import math
from typing import Any

import torch

from visionrl_b200.ops import _ext


def adamw_flat_reference(param, grad, master, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps,
                         weight_decay, step, clip_coef=None):
    g = grad.float()
    if clip_coef is not None:
        g = g * clip_coef
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    master.mul_(1 - lr * weight_decay).addcdiv_(exp_avg / bc1, denom, value=-lr)
    if param.data_ptr() != master.data_ptr():
        param.copy_(master)


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self._flat: list[dict[str, Any]] = []
        self._built = False
        self._shard_rank, self._shard_world = 0, 1
        self._allocator = None

    def set_shard(self, rank: int, world: int) -> None:
        """Keep master weights and moments only for slice ``rank`` of ``world`` equal slices of
        every flat buffer (optimiser-state sharding).  Must be called before the first step."""
        if self._built:
            raise RuntimeError("set_shard must be called before the flat buffers are built")
        self._shard_rank, self._shard_world = int(rank), int(world)

    def set_allocator(self, allocator) -> None:
        """``allocator(numel, dtype, device, tag)`` → 1-D tensor; lets the flat parameter and
        gradient buffers live in peer-mapped symmetric memory."""
        if self._built:
            raise RuntimeError("set_allocator must be called before the flat buffers are built")
        self._allocator = allocator

    # -- flat storage ------------------------------------------------------------------
    def _build(self) -> None:
        self._flat = []
        for group in self.param_groups:
            params = [p for p in group["params"]
                      if p.requires_grad and getattr(p, "_vrl_sharded", None) is None]
            by_key: dict[tuple, list] = {}
            for p in params:
                by_key.setdefault((p.device, p.dtype), []).append(p)
            for (device, dtype), plist in by_key.items():
                sizes = [p.numel() for p in plist]
                # 8-element alignment keeps every view 16-byte aligned in bf16
                offsets, total = [], 0
                for n in sizes:
                    offsets.append(total)
                    total += (n + 7) // 8 * 8
                world = self._shard_world
                total = (total + 8 * world - 1) // (8 * world) * (8 * world)
                if self._allocator is not None:
                    flat_p = self._allocator(total, dtype, device, "param").zero_()
                    flat_g = self._allocator(total, dtype, device, "grad").zero_()
                else:
                    flat_p = torch.zeros(total, device=device, dtype=dtype)
                    flat_g = torch.zeros(total, device=device, dtype=dtype)
                shard = total // world
                lo = self._shard_rank * shard
                for p, off in zip(plist, offsets):
                    n = p.numel()
                    flat_p[off:off + n].copy_(p.data.reshape(-1))
                    old_grad = p.grad
                    p.data = flat_p[off:off + n].view_as(p.data)
                    if old_grad is not None:
                        flat_g[off:off + n].copy_(old_grad.reshape(-1))
                    p.grad = flat_g[off:off + n].view_as(p.data)
                own = flat_p[lo:lo + shard]
                entry = dict(group=group, params=plist, offsets=offsets, sizes=sizes, param=flat_p,
                             grad=flat_g, exp_avg=torch.zeros(shard, device=device),
                             exp_avg_sq=torch.zeros(shard, device=device),
                             master=own if dtype == torch.float32 else own.float(), step=0,
                             total=total, shard=shard, lo=lo)
                self._flat.append(entry)
        self._built = True

    def _ensure(self) -> None:
        if not self._built:
            self._build()
            return
        for e in self._flat:
            for p, off in zip(e["params"], e["offsets"]):
                if p.data.data_ptr() != e["param"][off:].data_ptr() or p.device != e["param"].device:
                    self._rebuild_after_move()
                    return
                if p.grad is None or p.grad.data_ptr() != e["grad"][off:].data_ptr():
                    n = p.numel()
                    if p.grad is not None:
                        e["grad"][off:off + n].copy_(p.grad.reshape(-1))
                    p.grad = e["grad"][off:off + n].view_as(p.data)

    def _rebuild_after_move(self) -> None:
        """Parameters were moved (``model.to(...)``): re-flatten, keep moments and step."""
        old = self._flat
        self._build()
        for new, prev in zip(self._flat, old):
            dev = new["param"].device
            new["exp_avg"] = prev["exp_avg"].to(dev)
            new["exp_avg_sq"] = prev["exp_avg_sq"].to(dev)
            if new["param"].dtype != torch.float32:
                new["master"] = prev["master"].to(dev)
            else:
                new["master"] = new["param"][new["lo"]:new["lo"] + new["shard"]]
            new["step"] = prev["step"]

    def flat_buffers(self) -> list[dict[str, Any]]:
        self._ensure()
        return self._flat

    # -- optimiser API ---------------------------------------------------------------------
    @torch.no_grad()
    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of all gradients as a 0-d tensor on the parameters' device."""
        self._ensure()
        total = None
        for e in self._flat:
            g = e["grad"]
            if g.is_cuda and _ext.kernels_enabled():
                sq = _ext.load().sum_squares(g)
            else:
                sq = g.float().pow(2).sum()
            total = sq if total is None else total + sq.to(total.device)
        if total is None:
            return torch.zeros(())
        return total.sqrt()

    @torch.no_grad()
    def step(self, closure=None, clip_coef: torch.Tensor | None = None):
        loss = closure() if closure is not None else None
        self._ensure()
        for e in self._flat:
            g = e["group"]
            e["step"] += 1
            b1, b2 = g["betas"]
            kw = dict(lr=float(g["lr"]), beta1=float(b1), beta2=float(b2), eps=float(g["eps"]),
                      weight_decay=float(g["weight_decay"]), step=int(e["step"]))
            lo, n = e["lo"], e["shard"]
            p_own = e["param"][lo:lo + n]
            g_own = e.get("grad_shard")
            if g_own is None:
                g_own = e["grad"][lo:lo + n]
            if p_own.is_cuda and _ext.kernels_enabled():
                _ext.load().adamw_flat(p_own, g_own, e["master"], e["exp_avg"],
                                       e["exp_avg_sq"], kw["lr"], kw["beta1"], kw["beta2"],
                                       kw["eps"], kw["weight_decay"], kw["step"], clip_coef)
            else:
                adamw_flat_reference(p_own, g_own, e["master"], e["exp_avg"],
                                     e["exp_avg_sq"], clip_coef=clip_coef, **kw)
        return loss

    def zero_grad(self, set_to_none: bool = False) -> None:
        if not self._built:
            return super().zero_grad(set_to_none=True)
        for e in self._flat:
            e["grad"].zero_()

    # -- torch.optim.AdamW-compatible (de)serialisation ---------------------------------------
    def state_dict(self) -> dict[str, Any]:
        index = {}
        i = 0
        for group in self.param_groups:
            for p in group["params"]:
                index[id(p)] = i
                i += 1
        state: dict[int, dict[str, Any]] = {}
        for e in self._flat:
            full_m, full_v = self._full_moments(e)
            full_w = self._full_master(e)
            for p, off, n in zip(e["params"], e["offsets"], e["sizes"]):
                entry = {
                    "step": torch.tensor(float(e["step"])),
                    "exp_avg": full_m[off:off + n].view(p.shape).clone(),
                    "exp_avg_sq": full_v[off:off + n].view(p.shape).clone(),
                }
                if full_w is not None:
                    entry["master"] = full_w[off:off + n].view(p.shape).clone()
                state[index[id(p)]] = entry
        for group in self.param_groups:
            for p in group["params"]:
                handle = getattr(p, "_vrl_sharded", None)
                if handle is None or not p.requires_grad:
                    continue
                rt = handle.rt
                state[index[id(p)]] = {
                    "step": torch.tensor(float(rt.step_count)),
                    "exp_avg": rt.gather_state(handle, "exp_avg"),
                    "exp_avg_sq": rt.gather_state(handle, "exp_avg_sq"),
                    "master": rt.gather_state(handle, "master"),
                }
        groups = []
        start = 0
        for group in self.param_groups:
            g = {k: v for k, v in group.items() if k != "params"}
            g["params"] = list(range(start, start + len(group["params"])))
            start += len(group["params"])
            groups.append(g)
        return {"state": state, "param_groups": groups}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        saved_groups = state_dict["param_groups"]
        if len(saved_groups) != len(self.param_groups):
            raise ValueError("loaded state dict has a different number of parameter groups")
        for g, s in zip(self.param_groups, saved_groups):
            if len(g["params"]) != len(s["params"]):
                raise ValueError("loaded state dict contains a parameter group that doesn't match "
                                 "the size of optimizer's group")
            for k, v in s.items():
                if k != "params":
                    g[k] = v
        self._ensure()
        index = {}
        i = 0
        for group in self.param_groups:
            for p in group["params"]:
                index[id(p)] = i
                i += 1
        saved = {int(k): v for k, v in state_dict["state"].items()}
        for e in self._flat:
            for p, off, n in zip(e["params"], e["offsets"], e["sizes"]):
                s = saved.get(index[id(p)])
                if s is None:
                    continue
                if tuple(s["exp_avg"].shape) != tuple(p.shape):
                    raise ValueError("optimizer state shape does not match parameter shape")
                self._load_slice(e, "exp_avg", off, n, s["exp_avg"].reshape(-1))
                self._load_slice(e, "exp_avg_sq", off, n, s["exp_avg_sq"].reshape(-1))
                e["step"] = int(float(s["step"]))
            if e["param"].dtype != torch.float32:
                # bf16 rounding of the parameters is the fallback; a saved fp32 master wins
                e["master"].copy_(e["param"][e["lo"]:e["lo"] + e["shard"]])
                for p, off, n in zip(e["params"], e["offsets"], e["sizes"]):
                    s = saved.get(index[id(p)])
                    if s is not None and "master" in s:
                        self._load_slice(e, "master", off, n, s["master"].reshape(-1).float())
        for group in self.param_groups:
            for p in group["params"]:
                handle = getattr(p, "_vrl_sharded", None)
                s = saved.get(index.get(id(p), -1))
                if handle is None or s is None:
                    continue
                rt = handle.rt
                if tuple(s["exp_avg"].shape) != (handle.n, handle.k):
                    raise ValueError("optimizer state shape does not match the sharded weight's "
                                     f"full shape {(handle.n, handle.k)}")
                rt.load_state(handle, "exp_avg", s["exp_avg"])
                rt.load_state(handle, "exp_avg_sq", s["exp_avg_sq"])
                if "master" in s:
                    rt.load_state(handle, "master", s["master"])
                rt.step_count = int(float(s["step"]))

    @staticmethod
    def _load_slice(e, key: str, off: int, n: int, src: torch.Tensor) -> None:
        """Copy the part of a full-length parameter slice ``[off, off+n)`` owned by this shard."""
        lo, hi = e["lo"], e["lo"] + e["shard"]
        a, b = max(off, lo), min(off + n, hi)
        if a < b:
            e[key][a - lo:b - lo].copy_(src[a - off:b - off])

    def _full_master(self, e):
        """Full-length fp32 master weights, or ``None`` when the parameters are fp32 themselves."""
        if e["param"].dtype == torch.float32:
            return None
        if self._shard_world == 1:
            return e["master"]
        import torch.distributed as dist

        parts = [torch.empty_like(e["master"]) for _ in range(self._shard_world)]
        dist.all_gather(parts, e["master"].contiguous())
        return torch.cat(parts)

    def _full_moments(self, e):
        """Full-length moments (all shards, gathered when the state is sharded)."""
        if self._shard_world == 1:
            return e["exp_avg"], e["exp_avg_sq"]
        import torch.distributed as dist

        outs = []
        for key in ("exp_avg", "exp_avg_sq"):
            parts = [torch.empty_like(e[key]) for _ in range(self._shard_world)]
            dist.all_gather(parts, e[key].contiguous())
            outs.append(torch.cat(parts))
        return outs[0], outs[1]
