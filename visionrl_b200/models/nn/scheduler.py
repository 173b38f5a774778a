"""Flow-matching Euler schedule.

``set_timesteps(n)`` builds ``sigma_i`` on a linear grid from 1 to ``1/num_train``,
warps it with ``shift`` (``s*sigma / (1 + (s-1)*sigma)``), exposes
``timesteps = sigma * num_train`` and appends a trailing ``0`` to ``sigmas`` — the
interface :func:`visionrl_b200.algorithms.flow_matching.sde_step_with_logprob`
consumes (``sigmas``, ``index_for_timestep``).
"""

from __future__ import annotations

import torch


class FlowMatchEulerScheduler:
    order = 1

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 3.0):
        self.num_train_timesteps = num_train_timesteps
        self.shift = shift
        self.sigmas = torch.zeros(1)
        self.timesteps = torch.zeros(0)
        self.set_timesteps(num_train_timesteps)

    def set_timesteps(self, num_inference_steps: int, device=None) -> None:
        n = int(num_inference_steps)
        sigma = torch.linspace(1.0, 1.0 / self.num_train_timesteps, n, dtype=torch.float64)
        sigma = self.shift * sigma / (1 + (self.shift - 1) * sigma)
        self.timesteps = (sigma * self.num_train_timesteps).to(torch.float32)
        self.sigmas = torch.cat([sigma, sigma.new_zeros(1)]).to(torch.float32)
        if device is not None:
            self.timesteps = self.timesteps.to(device)
            self.sigmas = self.sigmas.to(device)

    def index_for_timestep(self, timestep) -> int:
        t = float(timestep)
        return int(torch.argmin((self.timesteps.float().cpu() - t).abs()).item())

    def indices_for_timesteps(self, timesteps) -> torch.Tensor:
        """Vectorised :meth:`index_for_timestep` that stays on the tensors' device."""
        ts = torch.as_tensor(timesteps, dtype=torch.float32, device=self.timesteps.device).reshape(-1)
        return torch.argmin((ts[:, None] - self.timesteps[None].float()).abs(), dim=1)

    def scale_noise(self, sample, timestep, noise):
        idx = self.indices_for_timesteps(timestep).to(sample.device)
        sigma = self.sigmas.to(sample.device)[idx].view(-1, *([1] * (sample.ndim - 1)))
        return (1.0 - sigma) * sample + sigma * noise

    def state(self) -> dict:
        return {"num_train_timesteps": self.num_train_timesteps, "shift": self.shift,
                "num_steps": int(self.timesteps.numel())}
