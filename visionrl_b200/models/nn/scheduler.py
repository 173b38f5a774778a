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


class DDPMNoiseScheduler:
    """Discrete variance-preserving forward process for the ``epsilon`` / ``v_prediction`` targets
    of the preference trainer (reference: ``vrl/trainers/offline_dpo.py:249-263`` calls
    ``add_noise`` / ``get_velocity`` on whatever scheduler it is given).

    ``alpha_bar_t`` is the running product of ``1 - beta_t`` with ``beta`` on the scaled-linear
    grid ``linspace(sqrt(b0), sqrt(b1), N) ** 2``; ``x_t = sqrt(alpha_bar_t) x_0 +
    sqrt(1 - alpha_bar_t) eps`` and ``v_t = sqrt(alpha_bar_t) eps - sqrt(1 - alpha_bar_t) x_0``.
    ``timesteps`` holds the integer steps in descending order, as a sampler would visit them.
    """

    order = 1

    def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.00085,
                 beta_end: float = 0.012, prediction_type: str = "epsilon"):
        from types import SimpleNamespace

        self.num_train_timesteps = int(num_train_timesteps)
        self.prediction_type = prediction_type
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, self.num_train_timesteps,
                               dtype=torch.float64) ** 2
        self.alphas_cumprod = torch.cumprod(1.0 - betas, dim=0).to(torch.float32)
        self.config = SimpleNamespace(num_train_timesteps=self.num_train_timesteps,
                                      prediction_type=prediction_type)
        self.timesteps = torch.zeros(0, dtype=torch.long)
        self.set_timesteps(self.num_train_timesteps)

    def set_timesteps(self, num_inference_steps: int, device=None) -> None:
        n = int(num_inference_steps)
        if not 1 <= n <= self.num_train_timesteps:
            raise ValueError(f"num_inference_steps must be in [1, {self.num_train_timesteps}], got {n}")
        stride = self.num_train_timesteps // n
        self.timesteps = (torch.arange(n, dtype=torch.long) * stride).flip(0)
        if device is not None:
            self.timesteps = self.timesteps.to(device)

    def _factors(self, sample: torch.Tensor, timesteps: torch.Tensor):
        t = torch.as_tensor(timesteps, device=sample.device).long().reshape(-1)
        if int(t.min()) < 0 or int(t.max()) >= self.num_train_timesteps:
            raise ValueError("timesteps out of range for this schedule")
        a = self.alphas_cumprod.to(sample.device)[t].view(-1, *([1] * (sample.ndim - 1)))
        return a.sqrt().to(sample.dtype), (1.0 - a).sqrt().to(sample.dtype)

    def add_noise(self, sample: torch.Tensor, noise: torch.Tensor, timesteps: torch.Tensor) -> torch.Tensor:
        keep, mix = self._factors(sample, timesteps)
        return keep * sample + mix * noise

    def get_velocity(self, sample: torch.Tensor, noise: torch.Tensor, timesteps: torch.Tensor) -> torch.Tensor:
        keep, mix = self._factors(sample, timesteps)
        return keep * noise - mix * sample

    def state(self) -> dict:
        return {"num_train_timesteps": self.num_train_timesteps, "prediction_type": self.prediction_type,
                "num_steps": int(self.timesteps.numel())}
