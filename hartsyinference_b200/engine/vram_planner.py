"""Per-phase decision whether a component's weights stay resident on the device or ride the block
streamer, with the numbers behind the decision in the log.

A generation has phases (text encode, denoise, VAE decode) whose peak is weights + activations. Only
the weight term can be streamed; a phase whose peak is activations needs a smaller working set
(tiled VAE decode, capped workspaces) instead, and the log line makes the two distinguishable.
Free memory is read after returning the caching allocator's unused blocks to the driver: memory
that was freed a moment ago (a text encoder released before the denoise phase) would otherwise count
as used and bias the plan towards streaming, which is several times slower.

Modes (flag ``low_vram`` / ``EngineOptions.low_vram``): ``auto`` measures and streams only what does
not fit, ``on`` streams whatever can be streamed (tests of the streamed path, shared GPUs), ``off``
never streams (an oversized model then fails loudly).

Reference: src/HartsyInference.Core/MemoryManagement/VramPlanner.cs (PlanPhase),
LowVramMode.cs (three-state policy), ResidentPrefixSizing.cs.
"""
from __future__ import annotations

import enum
from typing import Callable, Optional

import torch

from .. import config, log


class LowVramMode(str, enum.Enum):
    AUTO = "auto"
    ON = "on"
    OFF = "off"


class Placement(str, enum.Enum):
    RESIDENT = "resident"
    STREAMED = "streamed"


def resolve_mode(option=None) -> LowVramMode:
    """``option``: EngineOptions.low_vram (bool or mode name) when the caller set one, else the flag."""
    v = option if option not in (None, False) else config.get("low_vram")
    if isinstance(v, LowVramMode):
        return v
    if v is True or str(v).lower() in ("1", "true", "on", "yes"):
        return LowVramMode.ON
    if str(v).lower() in ("off", "never"):
        return LowVramMode.OFF
    return LowVramMode.AUTO


def resident_prefix(free_bytes: int, headroom_bytes: int, block_bytes: int, block_count: int) -> int:
    """Whole blocks that fit once the headroom is set aside, clamped to [0, block_count]."""
    if block_count < 0:
        raise ValueError("block_count")
    return max(0, min(block_count, (free_bytes - headroom_bytes) // max(block_bytes, 1)))


def _mb(n: int) -> str:
    return f"{n / 2**20:.0f} MB"


class VramPlanner:
    def __init__(self, device, model_name: str, mode: Optional[LowVramMode] = None,
                 free_bytes: Optional[Callable[[], int]] = None):
        self.device = torch.device(device)
        self.model_name = model_name
        self.mode = mode or resolve_mode()
        self._free = free_bytes

    @property
    def can_stream(self) -> bool:
        return self.device.type == "cuda" and self.mode != LowVramMode.OFF

    def available(self) -> int:
        """Free device bytes after handing the allocator's cached blocks back."""
        if self._free is not None:
            return int(self._free())
        if self.device.type != "cuda":
            return 1 << 62
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()
        return int(torch.cuda.mem_get_info(self.device)[0])

    def plan_phase(self, phase: str, weight_bytes: int, activation_bytes: int, already_resident: bool = False,
                   can_stream: bool = True) -> Placement:
        if weight_bytes < 0 or activation_bytes < 0:
            raise ValueError("negative size")
        what = f"weights {_mb(weight_bytes)}, activations {_mb(activation_bytes)}"
        tag = f"{self.model_name}/{phase}"
        if self.mode == LowVramMode.OFF:
            log.decision("VRAM", f"{tag}: resident (low_vram=off). {what}")
            return Placement.RESIDENT
        if already_resident:
            log.decision("VRAM", f"{tag}: resident (already on the device). {what}")
            return Placement.RESIDENT
        if self.device.type != "cuda" or not can_stream:
            why = "no device memory to plan" if self.device.type != "cuda" else "this model exposes no streamable blocks here"
            log.decision("VRAM", f"{tag}: resident ({why}). {what}")
            return Placement.RESIDENT
        free = self.available()
        if self.mode == LowVramMode.ON:
            log.decision("VRAM", f"{tag}: streamed (low_vram=on forces it). {what}, free {_mb(free)}")
            return Placement.STREAMED
        if weight_bytes + activation_bytes <= free:
            log.decision("VRAM", f"{tag}: resident. {what}, free {_mb(free)}")
            return Placement.RESIDENT
        if activation_bytes > free:
            log.decision("VRAM", f"{tag}: streamed, but the activations alone ({_mb(activation_bytes)}) exceed the free {_mb(free)}: "
                                 f"this phase needs a smaller working set (tiling), streaming only moves the weights")
        else:
            log.decision("VRAM", f"{tag}: streamed. {what} do not fit the free {_mb(free)}")
        return Placement.STREAMED


def checkpoint_bytes(ck, fp8: bool = False, shard: int = 1) -> int:
    """Bytes of a checkpoint's tensors as they will sit on the device: 2-D weights whose inner size is a
    multiple of 128 become one byte per value with ``fp8`` and are divided over ``shard`` ranks; the
    rest stays bf16."""
    total = 0
    for fobj in getattr(ck, "files", {}).values():
        for k in fobj.keys():
            _, shape = fobj.info(k)
            n = 1
            for d in shape:
                n *= int(d)
            big = len(shape) == 2 and shape[1] % 128 == 0 and n >= (1 << 16)
            total += (n // shard if big else n) * (1 if (fp8 and big) else 2)
    return total
