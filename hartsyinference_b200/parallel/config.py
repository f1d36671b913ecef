"""Parallel layout record.

Extends the reference's ``PlacementConfig`` (src/HartsyInference.Core/Backends/PlacementConfig.cs:
15-63: ShardDevices, TextEncoderDevice, VaeDevice, CfgParallelDevice, ContextParallelDevices,
TensorParallelDegree, CacheKey) with the degrees that only make sense on an NVSwitch box:
sequence (Ulysses), expert and data parallel.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ParallelConfig:
    tp: int = 1            # tensor parallel degree
    sp: int = 1            # Ulysses sequence parallel degree (DiT)
    ep: int = 1            # expert parallel degree (MoE)
    cfg: int = 1           # 2 = cond / uncond branches on separate device groups
    pp: int = 1            # pipeline stages (layer split / DiT-block split), NCCL p2p
    dp: int = 1            # independent replicas
    text_encoder_device: int = -1   # -1 = same as the denoiser
    vae_device: int = -1

    @property
    def world_size(self) -> int:
        return self.tp * self.sp * self.cfg * self.pp * self.dp * (1 if self.ep <= self.tp * self.sp * self.dp else self.ep)

    @property
    def is_single(self) -> bool:
        return self.world_size == 1

    @property
    def cache_key(self) -> str:
        return f"tp{self.tp}-sp{self.sp}-ep{self.ep}-cfg{self.cfg}-pp{self.pp}-dp{self.dp}-te{self.text_encoder_device}-vae{self.vae_device}"

    def describe(self) -> str:
        parts = [f"{k}{v}" for k, v in (("tp", self.tp), ("sp", self.sp), ("ep", self.ep), ("cfg", self.cfg),
                                        ("pp", self.pp), ("dp", self.dp)) if v > 1]
        return "+".join(parts) if parts else "single"

    @staticmethod
    def parse(text: str) -> "ParallelConfig":
        """Parse ``"tp8"``, ``"sp4+cfg2"``, ``"tp2+pp2"`` ... (the inverse of :meth:`describe`)."""
        kw = {}
        if text and text != "single":
            for part in text.replace(",", "+").split("+"):
                part = part.strip().lower()
                for key in ("cfg", "tp", "sp", "ep", "pp", "dp"):
                    if part.startswith(key):
                        kw[key] = int(part[len(key):])
                        break
                else:
                    raise ValueError(f"unknown parallel spec '{part}'")
        return ParallelConfig(**kw)
