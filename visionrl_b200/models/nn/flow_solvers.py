"""Multistep ODE solvers for flow-matching models: DPM-Solver++(2M) and UniPC (B(h) = e^h − 1).

The model predicts the velocity ``v = ε − x₀`` of the path ``x_σ = (1 − σ) x₀ + σ ε``.  Both
solvers work on the data prediction ``x₀ = x_σ − σ v`` in the half-log-SNR variable
``λ = log((1 − σ) / σ)``, keep the last predictions and take second-order multistep updates
(first order on the first step and, for stability, on the last one, where ``σ → 0``).

Interface (the same for both, shaped after the flow solvers the official Wan sampler uses,
reference call site ``vrl/models/families/wan_2_1/official_policy.py:453-478``):

    scheduler.set_timesteps(num_steps, device=None, shift=None, sigmas=None)
    scheduler.timesteps            # [num_steps]  σ · num_train_timesteps
    scheduler.sigmas               # [num_steps + 1], trailing 0
    x = scheduler.step(model_output, t, x)     # one call per timestep, in order

Everything is fp32 tensor arithmetic on the sample's device; no step synchronises with the host.
"""

from __future__ import annotations

import math

import torch


def get_sampling_sigmas(num_steps: int, shift: float, num_train_timesteps: int = 1000) -> torch.Tensor:
    """``num_steps`` noise levels: the uniform grid ``1, 1 − 1/n, …, 1/n`` warped by ``shift``
    (``σ' = s σ / (1 + (s − 1) σ)``), without the trailing zero.  The steps are even in σ, which is
    what keeps a multistep extrapolation in λ well behaved down to the last step."""
    del num_train_timesteps
    n = int(num_steps)
    sigma = torch.linspace(1.0, 0.0, n + 1, dtype=torch.float64)[:n]
    return (shift * sigma / (1 + (shift - 1) * sigma)).to(torch.float32)


class _FlowMultistep:
    order = 2

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0, solver_order: int = 2,
                 lower_order_final: bool = True) -> None:
        if solver_order not in (1, 2):
            raise ValueError("solver_order must be 1 or 2")
        self.num_train_timesteps = int(num_train_timesteps)
        self.shift = float(shift)
        self.solver_order = int(solver_order)
        self.lower_order_final = bool(lower_order_final)
        self.sigmas = torch.zeros(1)
        self.timesteps = torch.zeros(0)
        self._reset()

    def _reset(self) -> None:
        self._step = 0
        self._history: list[torch.Tensor] = []       # data predictions, newest first
        self._last_sample: torch.Tensor | None = None

    def set_timesteps(self, num_inference_steps: int | None = None, device=None,
                      shift: float | None = None, sigmas=None) -> None:
        if sigmas is None:
            if num_inference_steps is None:
                raise ValueError("give num_inference_steps or sigmas")
            sigmas = get_sampling_sigmas(num_inference_steps, self.shift if shift is None else shift,
                                         self.num_train_timesteps)
        sig = torch.as_tensor(sigmas, dtype=torch.float32).reshape(-1)
        if sig.numel() == 0 or bool((sig[1:] >= sig[:-1]).any()) or float(sig[0]) > 1.0 or float(sig[-1]) <= 0:
            raise ValueError("sigmas must decrease strictly inside (0, 1]")
        self.sigmas = torch.cat([sig, sig.new_zeros(1)])
        self.timesteps = sig * self.num_train_timesteps
        if device is not None:
            self.sigmas, self.timesteps = self.sigmas.to(device), self.timesteps.to(device)
        self._reset()

    @property
    def step_index(self) -> int:
        return self._step

    def index_for_timestep(self, timestep) -> int:
        return int(torch.argmin((self.timesteps.float().cpu() - float(timestep)).abs()).item())

    # σ = 1 has λ = −∞; the sampling grids start at σ slightly below the shifted 1.0 only for
    # shift = 1, so clamp for the logarithm and let the first-order formulas take the limit
    @staticmethod
    def _lam(sigma: float) -> float:
        s = min(max(sigma, 1e-12), 1.0 - 1e-7)
        return math.log((1.0 - s) / s)

    def _order_now(self, i: int, n: int) -> int:
        order = min(self.solver_order, len(self._history))
        if self.lower_order_final and i == n - 1:
            order = 1
        return max(order, 1)

    def _to_x0(self, model_output: torch.Tensor, sample: torch.Tensor, sigma: float) -> torch.Tensor:
        return sample.float() - sigma * model_output.float()


class FlowDPMSolverMultistepScheduler(_FlowMultistep):
    """DPM-Solver++(2M) on the data prediction."""

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor) -> torch.Tensor:
        del timestep                          # steps are taken in grid order
        i, n = self._step, int(self.timesteps.numel())
        if i >= n:
            raise RuntimeError("step() called more often than there are timesteps")
        sig = self.sigmas.tolist() if i == 0 else self._sig_list
        self._sig_list = sig
        s_cur, s_next = sig[i], sig[i + 1]
        x0 = self._to_x0(model_output, sample, s_cur)
        self._history.insert(0, x0)
        del self._history[self.solver_order:]
        x = sample.float()
        if s_next <= 0.0:                      # λ → ∞: the update collapses onto the prediction
            out = x0 if self._order_now(i, n) == 1 or len(self._history) < 2 else x0
        else:
            lam_s, lam_t = self._lam(s_cur), self._lam(s_next)
            h = lam_t - lam_s
            a_t = 1.0 - s_next
            phi = math.expm1(-h)               # e^{-h} − 1
            out = (s_next / s_cur) * x - a_t * phi * x0
            if self._order_now(i, n) == 2:
                h_last = lam_s - self._lam(sig[i - 1])
                r0 = h_last / h
                d1 = (x0 - self._history[1]) / r0
                out = out - 0.5 * a_t * phi * d1
        self._step += 1
        return out.to(sample.dtype)


class FlowUniPCMultistepScheduler(_FlowMultistep):
    """UniPC with B(h) = e^h − 1: a second-order predictor whose result is corrected, one step
    later, with the model evaluation made at the predicted point (no extra model calls)."""

    def _coefficients(self, h: float, order: int, rks: list[float], corrector: bool) -> list[float]:
        hh = -h
        h_phi_1 = math.expm1(hh)
        b_h = h_phi_1
        h_phi_k = h_phi_1 / hh - 1.0
        fact = 1.0
        rows, rhs = [], []
        for k in range(1, order + 1):
            rows.append([r ** (k - 1) for r in rks])
            rhs.append(h_phi_k * fact / b_h)
            fact *= k + 1
            h_phi_k = h_phi_k / hh - 1.0 / fact
        if corrector:
            if order == 1:
                return [0.5]
            return torch.linalg.solve(torch.tensor(rows, dtype=torch.float64),
                                      torch.tensor(rhs, dtype=torch.float64)).tolist()
        if order == 2:
            return [0.5]
        if order == 1:
            return []
        return torch.linalg.solve(torch.tensor(rows, dtype=torch.float64)[:-1, :-1],
                                  torch.tensor(rhs, dtype=torch.float64)[:-1]).tolist()

    def _update(self, x: torch.Tensor, m0: torch.Tensor, older: list[tuple[float, torch.Tensor]],
                s_from: float, s_to: float, order: int, new_pred: torch.Tensor | None) -> torch.Tensor:
        """Shared body of predictor (``new_pred is None``) and corrector."""
        lam_0, lam_t = self._lam(s_from), self._lam(s_to)
        h = lam_t - lam_0
        a_t = 1.0 - s_to
        rks, d1s = [], []
        for s_i, m_i in older[:order - 1]:
            rk = (self._lam(s_i) - lam_0) / h
            rks.append(rk)
            d1s.append((m_i - m0) / rk)
        rks.append(1.0)
        phi_1 = math.expm1(-h)
        out = (s_to / s_from) * x - a_t * phi_1 * m0
        rho = self._coefficients(h, order, rks, corrector=new_pred is not None)
        acc = None
        for coef, d in zip(rho, d1s):
            acc = coef * d if acc is None else acc + coef * d
        if new_pred is not None:
            last = rho[-1] * (new_pred - m0)
            acc = last if acc is None else acc + last
        if acc is not None:
            out = out - a_t * phi_1 * acc
        return out

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor) -> torch.Tensor:
        del timestep
        i, n = self._step, int(self.timesteps.numel())
        if i >= n:
            raise RuntimeError("step() called more often than there are timesteps")
        if i == 0:
            self._sig_list = self.sigmas.tolist()
            self._sig_hist: list[float] = []
        sig = self._sig_list
        s_cur, s_next = sig[i], sig[i + 1]
        x = sample.float()
        x0 = self._to_x0(model_output, x, s_cur)
        # corrector: redo the step that produced `sample`, now knowing the model at its end point
        if i > 0 and self._last_sample is not None:
            order = min(self.solver_order, len(self._history))
            older = list(zip(self._sig_hist[1:], self._history[1:]))
            x = self._update(self._last_sample, self._history[0], older, self._sig_hist[0], s_cur,
                             order, new_pred=x0)
            x0 = self._to_x0(model_output, x, s_cur)
        self._history.insert(0, x0)
        self._sig_hist.insert(0, s_cur)
        del self._history[self.solver_order:]
        del self._sig_hist[self.solver_order:]
        self._last_sample = x
        if s_next <= 0.0:
            out = x0
        else:
            order = self._order_now(i, n)
            older = list(zip(self._sig_hist[1:], self._history[1:]))
            out = self._update(x, x0, older, s_cur, s_next, order, new_pred=None)
        self._step += 1
        return out.to(sample.dtype)


def retrieve_timesteps(scheduler: _FlowMultistep, num_inference_steps: int | None = None, device=None,
                       sigmas=None, **kwargs):
    """``(timesteps, num_steps)`` after configuring ``scheduler`` from a step count or explicit sigmas."""
    scheduler.set_timesteps(num_inference_steps, device=device, sigmas=sigmas, **kwargs)
    return scheduler.timesteps, int(scheduler.timesteps.numel())


__all__ = ["FlowDPMSolverMultistepScheduler", "FlowUniPCMultistepScheduler", "get_sampling_sigmas",
           "retrieve_timesteps"]
