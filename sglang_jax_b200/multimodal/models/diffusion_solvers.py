"""Flow-matching samplers of the diffusion stage (reference
`multimodal/models/diffusion_solvers/{flow_match_euler,unipc}`).

The transformer predicts the velocity `v = noise - x0` at noise level `sigma` (x_sigma =
(1 - sigma) x0 + sigma noise).  Both solvers walk sigma from 1 to 0 on a shifted schedule
`sigma' = shift * sigma / (1 + (shift - 1) * sigma)`."""

from __future__ import annotations

import torch


def shifted_sigmas(num_steps: int, shift: float = 1.0, device="cpu") -> torch.Tensor:
    s = torch.linspace(1.0, 0.0, num_steps + 1, device=device, dtype=torch.float32)
    return shift * s / (1 + (shift - 1) * s)


class FlowMatchEulerDiscreteScheduler:
    """First-order: `x <- x + (sigma_next - sigma) * v`."""

    def __init__(self, shift: float = 1.0, num_train_timesteps: int = 1000):
        self.shift = shift
        self.num_train_timesteps = num_train_timesteps
        self.sigmas = None
        self.step_index = 0

    def set_timesteps(self, num_steps: int, device="cpu"):
        self.sigmas = shifted_sigmas(num_steps, self.shift, device)
        self.timesteps = self.sigmas[:-1] * self.num_train_timesteps
        self.step_index = 0

    def step(self, velocity: torch.Tensor, sample: torch.Tensor) -> torch.Tensor:
        s, s_next = self.sigmas[self.step_index], self.sigmas[self.step_index + 1]
        self.step_index += 1
        return (sample.float() + (s_next - s) * velocity.float()).to(sample.dtype)


class UniPCMultistepScheduler:
    """Second-order multistep predictor-corrector in the data-prediction form (UniPC with the
    B(h) = h variant): every step converts the velocity into an x0 estimate, corrects the previous
    update with it, then predicts the next sample from the last two x0 estimates."""

    def __init__(self, shift: float = 1.0, num_train_timesteps: int = 1000, solver_order: int = 2):
        self.shift = shift
        self.num_train_timesteps = num_train_timesteps
        self.order = solver_order
        self.sigmas = None

    def set_timesteps(self, num_steps: int, device="cpu"):
        self.sigmas = shifted_sigmas(num_steps, self.shift, device)
        self.timesteps = self.sigmas[:-1] * self.num_train_timesteps
        self.step_index = 0
        self.x0_hist: list[torch.Tensor] = []
        self.last_sample = None

    @staticmethod
    def _lambda(sigma):
        # log-SNR of the flow-matching path: alpha = 1 - sigma
        return torch.log((1 - sigma).clamp_min(1e-8)) - torch.log(sigma.clamp_min(1e-8))

    def _update(self, x, x0_list, s_prev, s_cur, s_next):
        """Data-prediction multistep update from sigma `s_cur` to `s_next`."""
        a_next = 1 - s_next
        if s_next <= 0:
            return x0_list[-1]
        h = self._lambda(s_next) - self._lambda(s_cur)
        base = (s_next / s_cur) * x - a_next * torch.expm1(-h) * x0_list[-1]
        if len(x0_list) < 2 or self.order < 2 or s_prev is None:
            return base
        h0 = self._lambda(s_cur) - self._lambda(s_prev)
        r = h0 / h
        d1 = (x0_list[-1] - x0_list[-2]) / r
        return base - 0.5 * a_next * torch.expm1(-h) * d1

    def step(self, velocity: torch.Tensor, sample: torch.Tensor) -> torch.Tensor:
        i = self.step_index
        s_cur, s_next = self.sigmas[i], self.sigmas[i + 1]
        x = sample.float()
        x0 = x - s_cur * velocity.float()
        if self.last_sample is not None and i > 0 and self.order >= 2:
            # corrector: redo the previous step with the x0 that is now known at its end point
            s_pp = self.sigmas[i - 2] if i >= 2 else None
            hist = self.x0_hist[-2:] if len(self.x0_hist) >= 2 else self.x0_hist[-1:]
            pred = self._update(self.last_sample, hist, s_pp, self.sigmas[i - 1], s_cur)
            a = 1 - s_cur
            h = self._lambda(s_cur) - self._lambda(self.sigmas[i - 1])
            x = pred - 0.5 * a * torch.expm1(-h) * (x0 - self.x0_hist[-1])
            x0 = x - s_cur * velocity.float()
        self.x0_hist.append(x0)
        self.x0_hist = self.x0_hist[-self.order:]
        s_prev = self.sigmas[i - 1] if i >= 1 else None
        nxt = self._update(x, self.x0_hist, s_prev, s_cur, s_next)
        self.last_sample = x
        self.step_index += 1
        return nxt.to(sample.dtype)


SOLVERS = {"FlowMatchEulerDiscreteScheduler": FlowMatchEulerDiscreteScheduler,
           "UniPCMultistepScheduler": UniPCMultistepScheduler}
