"""VRAM planner: per-phase resident / streamed decisions against a stated amount of free memory."""
import pytest
import torch

from hartsyinference_b200.engine.vram_planner import LowVramMode, Placement, VramPlanner, resident_prefix, resolve_mode

GB = 1 << 30


def _planner(free_gb, mode=LowVramMode.AUTO):
    p = VramPlanner("cuda:0", "m", mode, free_bytes=lambda: int(free_gb * GB))
    return p


def test_auto_streams_only_what_does_not_fit():
    assert _planner(40).plan_phase("denoise", 24 * GB, 4 * GB) == Placement.RESIDENT
    assert _planner(20).plan_phase("denoise", 24 * GB, 4 * GB) == Placement.STREAMED
    # weights that are on the device already are never re-planned (the free figure cannot see past them)
    assert _planner(2).plan_phase("denoise", 24 * GB, 4 * GB, already_resident=True) == Placement.RESIDENT
    # a model without streamable blocks (a tensor-parallel shard) stays resident whatever the numbers
    assert _planner(2).plan_phase("denoise", 24 * GB, 4 * GB, can_stream=False) == Placement.RESIDENT


def test_modes():
    assert _planner(100, LowVramMode.ON).plan_phase("denoise", GB, GB) == Placement.STREAMED
    assert _planner(1, LowVramMode.OFF).plan_phase("denoise", 24 * GB, GB) == Placement.RESIDENT
    assert resolve_mode(True) == LowVramMode.ON and resolve_mode("off") == LowVramMode.OFF and resolve_mode("auto") == LowVramMode.AUTO
    assert VramPlanner("cpu", "m").plan_phase("denoise", 24 * GB, GB) == Placement.RESIDENT
    with pytest.raises(ValueError):
        _planner(1).plan_phase("x", -1, 0)


def test_resident_prefix_arithmetic():
    assert resident_prefix(10 * GB, 2 * GB, GB, 57) == 8
    assert resident_prefix(100 * GB, 2 * GB, GB, 57) == 57
    assert resident_prefix(1 * GB, 2 * GB, GB, 57) == 0


def test_streamed_construction_parks_blocks_on_the_host():
    from hartsyinference_b200.models.dit import flux as F
    tr = F.FluxTransformer(F.tiny_flux(), "cpu", stream_blocks=True)
    # on the CPU there is nothing to park; the streamers exist and the forward pass walks them
    assert getattr(tr, "_streamers", None) is not None
    g = torch.Generator().manual_seed(0)
    cfg = tr.cfg
    img, txt = torch.randn(1, 16, cfg.in_channels, generator=g), torch.randn(1, 6, cfg.context_dim, generator=g)
    ii, it = F.flux_ids(4, 4, 6)
    ref = F.FluxTransformer(F.tiny_flux(), "cpu")
    args = (img, txt, torch.tensor([0.6]), torch.randn(1, cfg.pooled_dim, generator=g), ii, it, torch.tensor([3.5]))
    assert torch.allclose(tr.forward(*args).float(), ref.forward(*args).float(), atol=1e-3)
