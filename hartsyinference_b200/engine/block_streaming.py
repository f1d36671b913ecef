"""Block streaming for models that do not fit on the device ("low VRAM" mode).

The transformer blocks live in pinned host memory; two device slots hold the block that is
computing and the one being fetched. ``block(i)`` returns block i on the device and starts the
host-to-device copy of block i + 1 on a side stream, so the copy overlaps the compute of block i.
Events order the copy stream against the compute stream in both directions (a slot is not
overwritten while kernels of its previous occupant may still run).

Reference: src/HartsyInference.Core/MemoryManagement/BlockStreamingController.cs (Prime:71,
BeforeBlockForward:83, EvictAll:110, TrimAfterStep:129) and
src/HartsyInference.Cuda/CudaStreamingWeightCache.cs (upload stream, events, pinned staging).
B200s have 180 GB, so this is off by default (``B200_LOW_VRAM``).
"""
from __future__ import annotations

import copy
from typing import Any, Optional, Sequence

import torch


def map_tensors(obj: Any, fn):
    """Copy of a nested structure (dataclasses, lists, tuples, dicts) with ``fn`` applied to tensors."""
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return type(obj)(map_tensors(x, fn) for x in obj)
    if isinstance(obj, dict):
        return {k: map_tensors(v, fn) for k, v in obj.items()}
    if hasattr(obj, "__dataclass_fields__"):
        new = copy.copy(obj)
        for k in obj.__dataclass_fields__:
            setattr(new, k, map_tensors(getattr(obj, k), fn))
        return new
    return obj


def tree_bytes(obj: Any) -> int:
    total = 0

    def add(t):
        nonlocal total
        total += t.numel() * t.element_size()
        return t

    map_tensors(obj, add)
    return total


class BlockStreamer:
    def __init__(self, blocks: Sequence[Any], device, slots: int = 2):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        pin = (lambda t: t.detach().cpu().pin_memory()) if self.cuda else (lambda t: t.detach().cpu())
        self.host = [map_tensors(b, pin) for b in blocks]
        self.slots = max(2, slots)
        self._resident: dict[int, Any] = {}            # block index -> device copy
        self._ready: dict[int, Optional[torch.cuda.Event]] = {}
        self._free_after: dict[int, Optional[torch.cuda.Event]] = {}   # slot reuse fence per evicted block
        self._copy_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.uploads = 0
        self.bytes_uploaded = 0
        self._order: dict[int, int] = {}               # upload order, oldest evicted first
        self._tick = 0

    def __len__(self) -> int:
        return len(self.host)

    def _upload(self, i: int) -> None:
        if i in self._resident or not (0 <= i < len(self.host)):
            return
        while len(self._resident) >= self.slots:
            self._evict(min(self._resident, key=lambda j: self._order.get(j, -1)))
        if self.cuda:
            # the slot's previous occupant may still be read by kernels on the compute stream
            self._copy_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._copy_stream):
                dev = map_tensors(self.host[i], lambda t: t.to(self.device, non_blocking=True))
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
            self._ready[i] = ev
        else:
            dev = self.host[i]
            self._ready[i] = None
        self._resident[i] = dev
        self._order[i] = self._tick
        self._tick += 1
        self.uploads += 1
        self.bytes_uploaded += tree_bytes(self.host[i])

    def _evict(self, i: int) -> None:
        self._resident.pop(i, None)
        self._ready.pop(i, None)

    def prime(self, first: int = 0) -> None:
        """Start fetching the first blocks before the forward pass begins."""
        self._order, self._tick = {}, 0
        for i in range(first, min(first + self.slots, len(self.host))):
            self._upload(i)

    def block(self, i: int) -> Any:
        """Block i on the device (waits for its copy), and prefetch of block i + 1."""
        self._upload(i)
        ev = self._ready.get(i)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            self._ready[i] = None
        blk = self._resident[i]
        # everything older than the current block can go; then fetch the next one
        for j in [j for j in self._resident if j < i]:
            self._evict(j)
        self._upload(i + 1)
        return blk

    def evict_all(self) -> None:
        for j in list(self._resident):
            self._evict(j)
        if self.cuda:
            torch.cuda.current_stream(self.device).synchronize()
