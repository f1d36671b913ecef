"""Cheap RGB previews of latents during denoising.

A per-family linear map latents -> RGB (one 3 x C matrix and a bias applied per latent pixel) is what
preview decoders in image UIs use between steps; here the map is not a shipped table but is fitted
once per pipeline against the pipeline's own VAE: a few random latents are decoded, the images are
average-pooled to latent resolution, and the map is the least-squares solution. A preview then costs
one small matrix product instead of a VAE decode.

Reference: src/HartsyInference.Diffusion/Utilities/ (latent previews for the step callback;
the reference ships per-family factor tables and TAESD decoders).
"""
from __future__ import annotations

from typing import Optional

import torch


class LatentPreviewer:
    def __init__(self, factors: torch.Tensor, bias: torch.Tensor):
        self.factors, self.bias = factors.float(), bias.float()          # [C, 3], [3]

    @staticmethod
    def fit(vae, channels: int, samples: int = 3, size: int = 24, seed: int = 0) -> "LatentPreviewer":
        """Least-squares map from latent pixels to the VAE's (pooled) RGB output."""
        g = torch.Generator().manual_seed(seed)
        xs, ys = [], []
        for _ in range(samples):
            z = torch.randn(1, channels, size, size, generator=g)
            img = vae.decode(z).float().cpu()                                            # [1, 3, f * size, f * size] in [-1, 1]
            f = img.shape[-1] // size
            pooled = torch.nn.functional.avg_pool2d(img, f)[0]                            # [3, size, size]
            xs.append(z[0].reshape(channels, -1).t())
            ys.append(pooled.reshape(3, -1).t())
        x = torch.cat(xs)
        y = torch.cat(ys)
        xa = torch.cat([x, torch.ones(x.shape[0], 1)], 1)
        sol = torch.linalg.lstsq(xa, y).solution                                           # [C + 1, 3]
        return LatentPreviewer(sol[:-1], sol[-1])

    def rgb(self, latents: torch.Tensor) -> tuple[bytes, int, int]:
        """latents [1, C, h, w] (or [C, h, w]) -> (RGB24 bytes, width, height) at latent resolution."""
        z = latents.float().cpu()
        if z.ndim == 4:
            z = z[0]
        c, h, w = z.shape
        img = (z.reshape(c, -1).t() @ self.factors + self.bias).reshape(h, w, 3)
        u8 = ((img.clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)
        return u8.numpy().tobytes(), w, h


def in_guidance_interval(step: int, steps: int, interval: Optional[tuple]) -> bool:
    """Classifier-free guidance is applied on the steps whose position in [0, 1) lies inside
    ``interval`` = (start, end); None = always. Outside it only the conditional branch runs."""
    if not interval:
        return True
    lo, hi = float(interval[0]), float(interval[1])
    pos = step / max(steps, 1)
    return lo <= pos < hi or (hi >= 1.0 and pos >= lo)
