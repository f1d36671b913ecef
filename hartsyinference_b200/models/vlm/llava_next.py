"""LLaVA-NeXT: LLaVA with "any resolution" image handling.

An image is shown to the vision tower several times: once squeezed to the tower's input size, and
as the tiles of a higher-resolution canvas chosen from a list of allowed sizes (the one that keeps
the most of the image's pixels with the least padding). The tiles' patch features are laid back out
as one feature map, the rows / columns that only cover padding are cut off, a learned "newline"
embedding is appended to every feature row, and the result follows the base image's features.

Reference: src/HartsyInference.LLM/Multimodal/ (LLaVA-NeXT generator). Tensor names follow llava-hf
``LlavaNextForConditionalGeneration`` (``image_newline`` beside the LLaVA names).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from ..encoders.clip_vision import CLIP_MEAN, CLIP_STD, ClipVisionConfig
from ..llm.transformer import DecoderModel
from .llava import LlavaModel

DEFAULT_PINPOINTS = ((336, 672), (672, 336), (672, 672), (1008, 336), (336, 1008))


def select_best_resolution(size: tuple[int, int], pinpoints: Sequence[tuple[int, int]]) -> tuple[int, int]:
    """(height, width) of the canvas that keeps the most image pixels after an aspect-preserving
    fit; ties go to the canvas that wastes the least area."""
    h, w = size
    best, best_eff, best_waste = None, -1, None
    for ch, cw in pinpoints:
        s = min(cw / w, ch / h)
        eff = min(int(w * s) * int(h * s), w * h)
        waste = ch * cw - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (ch, cw), eff, waste
    return best


def _unpad(fmap: torch.Tensor, size: tuple[int, int]) -> torch.Tensor:
    """fmap [C, H, W] of a letter-boxed image -> the rows / columns that cover the image itself."""
    oh, ow = size
    ch, cw = fmap.shape[1:]
    if ow / oh > cw / ch:
        nh = int(round(oh * (cw / ow), 7))
        pad = (ch - nh) // 2
        return fmap[:, pad: ch - pad, :]
    nw = int(round(ow * (ch / oh), 7))
    pad = (cw - nw) // 2
    return fmap[:, :, pad: cw - pad]


class LlavaNextModel(LlavaModel):
    def __init__(self, decoder: DecoderModel, vision_cfg: ClipVisionConfig, image_token_id: int,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0, feature_layer: int = -2,
                 pinpoints: Sequence[tuple[int, int]] = DEFAULT_PINPOINTS):
        super().__init__(decoder, vision_cfg, image_token_id, get=get, seed=seed, feature_layer=feature_layer)
        self.pinpoints = [tuple(p) for p in pinpoints]
        H = decoder.cfg.hidden_size
        nl = get("image_newline") if get is not None else None
        if nl is None:
            if get is not None:
                raise KeyError("image_newline")
            nl = torch.randn(H, generator=torch.Generator().manual_seed(seed + 2)) * 0.02
        self.image_newline = nl.to(torch.bfloat16).to(self.device)

    def tiles(self, image: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int]]:
        """image [3, H, W] in [0, 1] -> (normalised views [1 + tiles, 3, S, S], (tile rows, tile columns)):
        the whole image squeezed to S x S, then the tiles of the letter-boxed best canvas."""
        S = self.vision.cfg.image_size
        _, h, w = image.shape
        ch, cw = select_best_resolution((h, w), self.pinpoints)
        s = min(cw / w, ch / h)
        nh, nw = min(int(h * s + 0.999999), ch), min(int(w * s + 0.999999), cw)      # ceil, as the processor does
        F = torch.nn.functional
        fit = F.interpolate(image[None].float(), size=(nh, nw), mode="bicubic", align_corners=False, antialias=True)[0].clamp(0, 1)
        top, left = (ch - nh) // 2, (cw - nw) // 2
        canvas = torch.zeros(3, ch, cw)
        canvas[:, top:top + nh, left:left + nw] = fit
        gh, gw = ch // S, cw // S
        tiles = canvas.reshape(3, gh, S, gw, S).permute(1, 3, 0, 2, 4).reshape(gh * gw, 3, S, S)
        base = F.interpolate(image[None].float(), size=(S, S), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
        views = torch.cat([base, tiles], 0)
        mean, std = torch.tensor(CLIP_MEAN)[None, :, None, None], torch.tensor(CLIP_STD)[None, :, None, None]
        return (views - mean) / std, (gh, gw)

    def pack(self, feats: torch.Tensor, grid: tuple[int, int], image_size: tuple[int, int]) -> torch.Tensor:
        """feats [1 + gh * gw, n, H] (base view first) -> [n + rows * (cols + 1), H]."""
        n = feats.shape[1]
        side = int(round(n ** 0.5))
        gh, gw = grid
        fmap = feats[1:].reshape(gh, gw, side, side, -1).permute(4, 0, 2, 1, 3).reshape(-1, gh * side, gw * side)
        fmap = _unpad(fmap, image_size)
        nl = self.image_newline.to(fmap.dtype)[:, None, None].expand(-1, fmap.shape[1], 1)
        fmap = torch.cat([fmap, nl], 2)
        return torch.cat([feats[0], fmap.flatten(1).t()], 0)

    @torch.no_grad()
    def image_features_anyres(self, image: torch.Tensor) -> torch.Tensor:
        """image [3, H, W] in [0, 1] (any size) -> the packed embeddings in the decoder's space."""
        views, grid = self.tiles(image)
        feats = torch.stack([self.image_features(v) for v in views])
        return self.pack(feats, grid, tuple(image.shape[1:]))

    def expand_prompt(self, token_ids: Sequence[int], images: Sequence[torch.Tensor]):
        """Like LLaVA's, with images given in [0, 1] at their own size: each image token becomes as
        many placeholders as that image's packed features."""
        feats = [self.image_features_anyres(im) for im in images]
        return self._splice(token_ids, feats)
