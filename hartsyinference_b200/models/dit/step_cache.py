"""First-block cache for DiT denoising loops.

Each step runs the first transformer block; if its output moved little since the previous step
(relative L1 change below a threshold, accumulated since the last full run) the remaining blocks
are skipped and the residual they produced last time is re-applied. The decision is made from a
device scalar read once per step; everything else stays on the device.

Reference: src/HartsyInference.Diffusion/Utilities/DeviceFeatureCache.cs (ShouldCompute:82,
StoreResidual:127, ApplyResidual:16x) and the ``step_cache_threshold`` engine flag.
"""
from __future__ import annotations

from typing import Optional

import torch


class FirstBlockCache:
    def __init__(self, threshold: float, max_consecutive_skips: int = 3):
        self.threshold = float(threshold)
        self.max_skips = max_consecutive_skips
        self.prev_first: Optional[torch.Tensor] = None
        self.residual: Optional[torch.Tensor] = None
        self.accum = 0.0
        self.skips_in_a_row = 0
        self.computed = 0
        self.skipped = 0

    @property
    def enabled(self) -> bool:
        return self.threshold > 0

    def reset(self) -> None:
        self.prev_first = self.residual = None
        self.accum, self.skips_in_a_row = 0.0, 0

    def should_compute(self, first_out: torch.Tensor) -> bool:
        """Call with the first block's output. True: run the remaining blocks and then
        :meth:`store_residual`; False: call :meth:`apply_residual`."""
        if not self.enabled or self.prev_first is None or self.residual is None \
                or self.prev_first.shape != first_out.shape:
            self.prev_first = first_out.detach().clone()
            self.accum, self.skips_in_a_row = 0.0, 0
            return True
        a, b = first_out.float(), self.prev_first.float()
        change = float(((a - b).abs().mean() / b.abs().mean().clamp_min(1e-12)).item())
        self.prev_first = first_out.detach().clone()
        self.accum += change
        if self.accum < self.threshold and self.skips_in_a_row < self.max_skips:
            self.skips_in_a_row += 1
            self.skipped += 1
            return False
        self.accum, self.skips_in_a_row = 0.0, 0
        return True

    def store_residual(self, first_out: torch.Tensor, final_out: torch.Tensor) -> None:
        self.residual = (final_out.float() - first_out.float()).to(final_out.dtype)
        self.computed += 1

    def apply_residual(self, first_out: torch.Tensor) -> torch.Tensor:
        return (first_out.float() + self.residual.float()).to(first_out.dtype)
