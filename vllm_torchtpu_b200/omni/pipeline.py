"""Sampling loop of a diffusion transformer: classifier-free guidance over a flow-matching schedule.

The conditional and unconditional branches of a step run as one batch of two (one pass through the
weights); per-step device times are kept with CUDA events and read after the loop, so the loop never waits
for the device (reference: the external omni runtime's generation worker; device-side timing in
src/vllm_torchtpu/omni/profiler.py)."""
from __future__ import annotations

from typing import Optional

import torch

from .dit import DiffusionTransformer, DiTConfig
from .scheduler import FlowMatchEulerScheduler


class DiffusionPipeline:
    def __init__(self, cfg: DiTConfig, device: str = "cuda", state_dict: Optional[dict] = None, shift: float = 3.0):
        self.cfg = cfg
        self.device = torch.device(device)
        self.model = DiffusionTransformer(cfg, device, state_dict)
        self.scheduler = FlowMatchEulerScheduler(shift=shift)
        self.step_ms: list = []

    @torch.no_grad()
    def generate(self, text: torch.Tensor, latent_shape: tuple, num_steps: int = 8, guidance_scale: float = 1.0,
                 negative_text: Optional[torch.Tensor] = None, seed: int = 0,
                 latents: Optional[torch.Tensor] = None) -> torch.Tensor:
        """text [B, L, text_dim]; latent_shape (C, F, H, W) -> denoised latents [B, C, F, H, W]."""
        B = text.shape[0]
        cfg_on = guidance_scale != 1.0
        if cfg_on and negative_text is None:
            negative_text = torch.zeros_like(text)
        if latents is None:
            g = torch.Generator().manual_seed(seed)
            latents = torch.randn((B, *latent_shape), generator=g, dtype=torch.float32)
        x = latents.to(device=self.device, dtype=self.cfg.dtype)
        text = text.to(self.device)
        both = torch.cat([text, negative_text.to(self.device)]) if cfg_on else text
        self.scheduler.set_timesteps(num_steps, self.device)
        cuda = self.device.type == "cuda"
        events = []
        for i, t in enumerate(self.scheduler.timesteps):
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            xin = torch.cat([x, x]) if cfg_on else x
            v = self.model.forward(xin, t.expand(xin.shape[0]), both)
            if cfg_on:
                vc, vu = v[:B].float(), v[B:].float()
                v = vu + guidance_scale * (vc - vu)
            x = self.scheduler.step(v, i, x)
            if cuda:
                e1.record()
                events.append((e0, e1))
        if cuda:
            torch.cuda.synchronize(self.device)
            self.step_ms = [a.elapsed_time(b) for a, b in events]
        return x
