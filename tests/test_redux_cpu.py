"""Flux Redux picture prompts: the projector's arithmetic and the way its tokens join the text states."""
import pytest
import torch
import torch.nn.functional as F

from hartsyinference_b200.models.dit.redux import ReduxImageEncoder


def test_projector_arithmetic_and_shapes():
    g = torch.Generator().manual_seed(0)
    w = {"redux_up.weight": torch.randn(36, 8, generator=g), "redux_up.bias": torch.randn(36, generator=g),
         "redux_down.weight": torch.randn(12, 36, generator=g), "redux_down.bias": torch.randn(12, generator=g)}
    r = ReduxImageEncoder(w.get)
    x = torch.randn(5, 8, generator=g)
    want = F.linear(F.silu(F.linear(x, w["redux_up.weight"], w["redux_up.bias"])), w["redux_down.weight"], w["redux_down.bias"])
    assert torch.allclose(r(x), want, atol=1e-6) and torch.allclose(r(x, 0.5), want * 0.5, atol=1e-6)
    with pytest.raises(ValueError):
        r(torch.randn(5, 9))
    full = ReduxImageEncoder(None, "meta")
    assert full.up[0].shape == (12288, 1152) and full.down[0].shape == (4096, 12288)        # the released projector


def test_pipeline_appends_picture_tokens():
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ImageRequest, Modality, ModelSpec
    eng = InferenceEngine("cpu")
    spec = ModelSpec("synthetic:flux-tiny", Modality.IMAGE)
    pipe = eng.images.pipeline(spec)
    tdim = pipe.c.transformer.cfg.context_dim
    req = dict(prompt="a fox", width=32, height=32, steps=2, seed=3)
    with pytest.raises(ValueError):
        pipe.generate(ImageRequest(image_prompt=torch.rand(3, 16, 16), **req))
    pipe.c.redux = ReduxImageEncoder(None, "cpu", in_dim=8, txt_dim=tdim, seed=1)
    seen = {}
    pipe.c.image_states = lambda picture: torch.full((6, 8), float(torch.as_tensor(picture).float().mean()))
    orig = pipe.denoise

    def spy(ctx, *a, **k):
        seen["rows"] = ctx.shape[0]
        return orig(ctx, *a, **k)

    pipe.denoise = spy
    plain = pipe.generate(ImageRequest(**req))
    rows = seen["rows"]
    with_picture = pipe.generate(ImageRequest(image_prompt=torch.rand(3, 16, 16), **req))
    assert seen["rows"] == rows + 6 and with_picture.rgb != plain.rgb
    other = pipe.generate(ImageRequest(image_prompt=torch.zeros(3, 16, 16), **req))
    assert other.rgb != with_picture.rgb
