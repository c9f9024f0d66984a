"""Flow-matching Euler scheduler (the sampler of Wan / Flux / Qwen-Image class models).

The model predicts a velocity v(x_t, t) = noise - data; a step moves the sample along it from sigma_i to
sigma_{i+1}.  Sigmas run from 1 (pure noise) to 0 and are warped by ``shift`` so that more steps are spent at
high noise for large images: sigma' = shift * sigma / (1 + (shift - 1) * sigma)."""
from __future__ import annotations

import torch


class FlowMatchEulerScheduler:
    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0):
        self.num_train_timesteps = num_train_timesteps
        self.shift = float(shift)
        self.sigmas = None
        self.timesteps = None

    def set_timesteps(self, num_steps: int, device="cpu") -> None:
        if num_steps < 1:
            raise ValueError("num_steps must be >= 1")
        s = torch.linspace(1.0, 1.0 / self.num_train_timesteps, num_steps, dtype=torch.float64)
        s = self.shift * s / (1 + (self.shift - 1) * s)
        self.timesteps = (s * self.num_train_timesteps).float().to(device)
        self.sigmas = torch.cat([s, s.new_zeros(1)]).float().to(device)

    def step(self, velocity: torch.Tensor, i: int, sample: torch.Tensor) -> torch.Tensor:
        dt = (self.sigmas[i + 1] - self.sigmas[i]).to(torch.float32)
        return (sample.float() + dt * velocity.float()).to(sample.dtype)

    def add_noise(self, data: torch.Tensor, noise: torch.Tensor, sigma: float) -> torch.Tensor:
        return ((1 - sigma) * data.float() + sigma * noise.float()).to(data.dtype)
