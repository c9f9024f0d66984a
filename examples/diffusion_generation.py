"""Latents of a Wan-style diffusion transformer with a flow-matching sampling loop.
`python examples/diffusion_generation.py --frames 2 --height 16 --width 16 --steps 8 --guidance-scale 3`
(random-init weights of a small configuration; `--device cpu` runs the fp32 statement without a GPU)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from vllm_torchtpu_b200.omni.dit import DiTConfig  # noqa: E402
from vllm_torchtpu_b200.omni.pipeline import DiffusionPipeline  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--frames", type=int, default=2)
    ap.add_argument("--height", type=int, default=16, help="latent rows (a multiple of 2)")
    ap.add_argument("--width", type=int, default=16, help="latent columns (a multiple of 2)")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--guidance-scale", type=float, default=3.0)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    cfg = DiTConfig(num_layers=a.layers, num_heads=a.heads, head_dim=a.head_dim, hidden_size=a.heads * a.head_dim,
                    ffn_dim=4 * a.heads * a.head_dim, dtype=torch.bfloat16 if a.device == "cuda" else torch.float32)
    pipe = DiffusionPipeline(cfg, a.device)
    text = torch.randn(1, 16, cfg.text_dim, generator=torch.Generator().manual_seed(a.seed))      # stands in for a text encoder
    lat = pipe.generate(text, (cfg.in_channels, a.frames, a.height, a.width), num_steps=a.steps,
                        guidance_scale=a.guidance_scale, seed=a.seed)
    tokens = a.frames * (a.height // 2) * (a.width // 2)
    print(f"latents {tuple(lat.shape)}  tokens per sample {tokens}  mean {float(lat.float().mean()):+.4f}  "
          f"std {float(lat.float().std()):.4f}")
    if pipe.step_ms:
        print("ms per step:", " ".join(f"{ms:.2f}" for ms in pipe.step_ms))
    return lat


if __name__ == "__main__":
    main()
