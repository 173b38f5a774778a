"""Exponential moving average of the trainable parameters.

``d_t = min((1 + t) / (10 + t), decay)``; every ``update_step_interval`` optimiser
steps (``(t + 1) % interval == 0``) the shadow moves by ``ema += (1 - d_t)(p - ema)``
(reference: ``vrl/trainers/ema.py:15-101``).  The update is a single fused
multi-tensor launch (``torch._foreach_lerp_``) instead of one kernel per parameter.
"""

from __future__ import annotations

from collections.abc import Iterable

import torch


class EMAModuleWrapper:
    def __init__(self, parameters: Iterable[torch.nn.Parameter], decay: float = 0.9999,
                 update_step_interval: int = 1, device: torch.device | str | None = None):
        params = list(parameters)
        self.decay = decay
        self.update_step_interval = max(1, int(update_step_interval))
        self.device = torch.device(device) if device is not None else None
        self.ema_parameters = [p.detach().clone().float().to(self.device or p.device) for p in params]
        self.temp_stored_parameters: list[torch.Tensor] | None = None

    def get_current_decay(self, optimization_step: int) -> float:
        return min((1 + optimization_step) / (10 + optimization_step), self.decay)

    @torch.no_grad()
    def step(self, parameters: Iterable[torch.nn.Parameter], optimization_step: int) -> None:
        params = list(parameters)
        if (optimization_step + 1) % self.update_step_interval != 0:
            return
        weight = 1.0 - self.get_current_decay(optimization_step)
        pairs = [(e, p) for e, p in zip(self.ema_parameters, params, strict=True) if p.requires_grad]
        if not pairs:
            return
        emas = [e for e, _ in pairs]
        src = [p.detach().to(device=e.device, dtype=e.dtype) for e, p in pairs]
        torch._foreach_lerp_(emas, src, weight)

    def to(self, device=None, dtype=None) -> None:
        self.device = torch.device(device) if device is not None else self.device
        self.ema_parameters = [e.to(device=device, dtype=dtype) if e.is_floating_point()
                               else e.to(device=device) for e in self.ema_parameters]

    @torch.no_grad()
    def copy_ema_to(self, parameters: Iterable[torch.nn.Parameter], store_temp: bool = True) -> None:
        params = list(parameters)
        if store_temp:
            self.temp_stored_parameters = [p.detach().cpu().clone() for p in params]
        for e, p in zip(self.ema_parameters, params, strict=True):
            p.data.copy_(e.to(p.device, p.dtype))

    @torch.no_grad()
    def copy_temp_to(self, parameters: Iterable[torch.nn.Parameter]) -> None:
        if self.temp_stored_parameters is None:
            raise RuntimeError("no stored parameters: call copy_ema_to(store_temp=True) first")
        for t, p in zip(self.temp_stored_parameters, parameters, strict=True):
            p.data.copy_(t.to(p.device, p.dtype))
        self.temp_stored_parameters = None

    def state_dict(self) -> dict:
        return {"decay": self.decay, "ema_parameters": [e.detach().cpu() for e in self.ema_parameters]}

    def load_state_dict(self, state_dict: dict) -> None:
        state = state_dict
        self.decay = state.get("decay", self.decay)
        loaded = state["ema_parameters"]
        if len(loaded) != len(self.ema_parameters):
            raise ValueError(f"EMA state has {len(loaded)} tensors, expected {len(self.ema_parameters)}")
        self.ema_parameters = [t.to(device=e.device, dtype=e.dtype)
                               for t, e in zip(loaded, self.ema_parameters)]
