"""Diffusion utilities: latent previews fitted against the VAE, guidance interval, tiled VAE decode."""
import torch

from hartsyinference_b200.engine.requests import ImageRequest, ModelSpec, Modality
from hartsyinference_b200.models.diffusion.preview import LatentPreviewer, in_guidance_interval
from hartsyinference_b200.models.vae.vae2d import Vae2dDecoder, tiny_vae2d


def test_guidance_interval_positions():
    assert all(in_guidance_interval(i, 10, None) for i in range(10))
    on = [i for i in range(10) if in_guidance_interval(i, 10, (0.2, 0.6))]
    assert on == [2, 3, 4, 5]
    assert [i for i in range(4) if in_guidance_interval(i, 4, (0.5, 1.0))] == [2, 3]


def test_previewer_recovers_a_linear_decoder():
    class Lin:
        """A 'VAE' whose output really is linear in the latents: the fit must reproduce it."""
        def __init__(self):
            g = torch.Generator().manual_seed(1)
            self.m = torch.randn(4, 3, generator=g) * 0.2
            self.b = torch.tensor([0.1, -0.2, 0.05])

        def decode(self, z):
            img = torch.einsum("bchw,cd->bdhw", z.float(), self.m) + self.b[None, :, None, None]
            return torch.nn.functional.interpolate(img, scale_factor=8, mode="nearest")

    v = Lin()
    p = LatentPreviewer.fit(v, 4)
    assert torch.allclose(p.factors, v.m, atol=1e-4) and torch.allclose(p.bias, v.b, atol=1e-4)
    rgb, w, h = p.rgb(torch.zeros(1, 4, 5, 7))
    assert (w, h) == (7, 5) and len(rgb) == 5 * 7 * 3


def test_tiled_decode_matches_full_decode_away_from_context_effects():
    torch.manual_seed(0)
    vae = Vae2dDecoder(tiny_vae2d(), "cpu", torch.float32)
    z = torch.randn(1, vae.cfg.latent_channels, 24, 20) * 0.5
    full = vae.decode(z)
    tiled = vae.decode_tiled(z, tile=16, overlap=8)
    assert tiled.shape == full.shape
    # tiles normalise over their own extent, so the two agree up to the tiling tolerance
    rel = float((tiled - full).norm() / full.norm())
    assert rel < 0.35, rel
    # and a latent no larger than a tile takes the plain path exactly
    assert torch.equal(vae.decode_tiled(z[:, :, :16, :16], tile=16, overlap=8), vae.decode(z[:, :, :16, :16]))


def test_pipeline_preview_and_tiling_options():
    from hartsyinference_b200.engine.inference_engine import InferenceEngine
    eng = InferenceEngine("cpu")
    seen = []
    res = eng.images.generate(ModelSpec("synthetic:flux-dev-tiny", Modality.IMAGE),
                              ImageRequest(prompt="a", negative_prompt="b", cfg_scale=2.0, guidance_interval=(0.0, 0.5), width=64,
                                           height=64, steps=4, seed=1, preview_every=2, vae_tile=4),
                              progress=lambda p: seen.append((p.step, p.preview_rgb is not None, p.preview_width, p.preview_height)))
    assert res.width == 64 and len(res.rgb) == 64 * 64 * 3
    assert seen == [(1, False, 0, 0), (2, True, 8, 8), (3, False, 0, 0), (4, True, 8, 8)]
