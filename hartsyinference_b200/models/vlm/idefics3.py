"""Idefics3 / SmolVLM vision-language models (SigLIP-style tower, pixel-shuffle connector, Llama-class
decoder).

An image is resized so that both sides are multiples of the tower's input size, cut into a grid of
tiles of that size, and followed by one down-scaled view of the whole picture. Every tile (and the
global view) runs through the vision tower; the connector folds each ``s x s`` neighbourhood of patch
states into one row (pixel shuffle) and projects it to the decoder width, so a tile costs
``(size / patch / s)^2`` rows of the prompt. In the prompt every tile is announced by
``<fake_token_around_image><row_R_col_C>`` (the global view by ``<fake_token_around_image><global-img>``)
and rows of tiles end with a newline, as the models were trained; the serving engine then prefills
the mixed text / image embeddings like for the other image-text models.

Reference: src/HartsyInference.LLM/Multimodal/ (image-text generators behind the text service; SmolVLM2
is one of the models of its scoreboard). Tensor names follow Hugging Face
``Idefics3ForConditionalGeneration`` / ``SmolVLMForConditionalGeneration``: ``model.vision_model.*``,
``model.connector.modality_projection.proj``, ``model.text_model.*``, ``lm_head``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F

from ... import ops
from ..dit.common import WeightFactory
from ..encoders.vit import VitConfig, VitEncoder
from ..llm.transformer import DecoderModel

MEAN = STD = 0.5


def idefics3_vision_from_hf(d: dict) -> VitConfig:
    width = int(d.get("hidden_size", 1152))
    act = d.get("hidden_act", "gelu_pytorch_tanh")
    return VitConfig(kind="siglip", image_size=int(d.get("image_size", 364)), patch=int(d.get("patch_size", 14)), width=width,
                     layers=int(d.get("num_hidden_layers", 27)), heads=int(d.get("num_attention_heads", 16)),
                     ffn=int(d.get("intermediate_size", 4304)), activation="gelu_tanh" if "tanh" in act else "gelu",
                     eps=float(d.get("layer_norm_eps", 1e-6)))


class Idefics3Model:
    image_prefix_ids: tuple = ()
    image_suffix_ids: tuple = ()

    def __init__(self, decoder: DecoderModel, vision_cfg: VitConfig, image_token_id: int, scale_factor: int = 2,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0, longest_edge: Optional[int] = None):
        self.decoder, self.device = decoder, decoder.device
        self.image_token_id = int(image_token_id)
        self.scale = int(scale_factor)
        self.vision = VitEncoder(vision_cfg, self.device, get=get, seed=seed, prefix="model.vision_model.")
        f = WeightFactory(self.device, False, get=get, seed=seed + 1)
        self.proj = f.linear("model.connector.modality_projection.proj", decoder.cfg.hidden_size, vision_cfg.width * self.scale ** 2, bias=False)
        self.tile = vision_cfg.image_size
        self.longest_edge = int(longest_edge or 4 * self.tile)
        grid = vision_cfg.image_size // vision_cfg.patch
        self.rows_per_tile = (grid // self.scale) ** 2
        # ids of the structure tokens; filled by ``bind_tokenizer`` (a checkpoint's own tokenizer has them)
        self.fake_id: Optional[int] = None
        self.global_id: Optional[int] = None
        self.newline_ids: list = []
        self._cell_ids: dict = {}
        self._token_id: Optional[Callable[[str], Optional[int]]] = None

    # ------------------------------------------------------------------------------ prompt structure
    def bind_tokenizer(self, token_id: Callable[[str], Optional[int]], newline_ids: Sequence[int]) -> None:
        """``token_id(text)`` -> id of a special token or None; ``newline_ids``: the encoding of "\\n"."""
        self._token_id = token_id
        self.fake_id = token_id("<fake_token_around_image>")
        self.global_id = token_id("<global-img>")
        self.newline_ids = list(newline_ids)

    def _cell(self, r: int, c: int) -> Optional[int]:
        key = (r, c)
        if key not in self._cell_ids:
            self._cell_ids[key] = self._token_id(f"<row_{r + 1}_col_{c + 1}>") if self._token_id else None
        return self._cell_ids[key]

    def image_block(self, rows: int, cols: int) -> list:
        """Token ids of one image: per tile ``<fake><row_R_col_C>`` + its image tokens, a newline after every
        row of tiles, then ``\\n<fake><global-img>`` + image tokens + ``<fake>``. Structure tokens the
        tokenizer does not know are left out."""
        img = [self.image_token_id] * self.rows_per_tile
        opt = lambda t: [] if t is None else [t]
        out: list = []
        for r in range(rows):
            for c in range(cols):
                out += opt(self.fake_id) + opt(self._cell(r, c)) + img
            out += self.newline_ids
        if rows:
            out += self.newline_ids
        return out + opt(self.fake_id) + opt(self.global_id) + img + opt(self.fake_id)

    # ------------------------------------------------------------------------------ images
    def split_image(self, image: torch.Tensor):
        """image [3, H, W] in [0, 1] -> (views [n, 3, S, S] normalised, tile rows, tile columns): the tiles in
        row-major order, then the global view. Pictures that fit one tile give the global view only."""
        s = self.tile
        _, h, w = image.shape
        k = self.longest_edge / max(h, w)
        h2, w2 = max(1, round(h * k)), max(1, round(w * k))
        if h2 <= s and w2 <= s:
            rows = cols = 0
            tiles = []
        else:
            rows, cols = math.ceil(h2 / s), math.ceil(w2 / s)
            big = F.interpolate(image[None].float(), size=(rows * s, cols * s), mode="bicubic", align_corners=False, antialias=True)[0]
            tiles = [big[:, r * s:(r + 1) * s, c * s:(c + 1) * s] for r in range(rows) for c in range(cols)]
        whole = F.interpolate(image[None].float(), size=(s, s), mode="bicubic", align_corners=False, antialias=True)[0]
        views = torch.stack(tiles + [whole]).clamp(0, 1)
        return (views - MEAN) / STD, rows, cols

    @torch.no_grad()
    def view_features(self, views: torch.Tensor) -> torch.Tensor:
        """views [n, 3, S, S] normalised -> [n * rows_per_tile, hidden] rows in the decoder's space."""
        out = []
        g = self.tile // self.vision.cfg.patch
        sf = self.scale
        for v in views:
            h = self.vision.hidden_states(v)                                   # [g * g, W], final LayerNorm applied
            wd = h.shape[-1]
            x = h.reshape(g // sf, sf, g // sf, sf, wd).permute(0, 2, 1, 3, 4).reshape((g // sf) ** 2, sf * sf * wd)
            out.append(ops.linear(x.contiguous(), self.proj))
        return torch.cat(out, 0)

    @torch.no_grad()
    def image_features_anyres(self, image: torch.Tensor) -> torch.Tensor:
        views, _, _ = self.split_image(image)
        return self.view_features(views)

    def expand_prompt(self, token_ids: Sequence[int], images: Sequence[torch.Tensor]):
        """Every image token of ``token_ids`` stands for one picture: it becomes that picture's block of
        structure tokens and image rows. Returns (ids, embeds [T, H], mask [T])."""
        ids: list = []
        rows_e: list = []
        mask: list = []
        it = iter(images)
        hdim = self.decoder.cfg.hidden_size
        zero = lambda n: torch.zeros(n, hdim, dtype=torch.bfloat16, device=self.device)
        for t in token_ids:
            if t != self.image_token_id:
                ids.append(int(t)); rows_e.append(zero(1)); mask.append(False)
                continue
            im = next(it, None)
            if im is None:
                raise ValueError("more image tokens than images")
            views, r, c = self.split_image(im)
            feats = self.view_features(views)
            at = 0
            for tok in self.image_block(r, c):
                ids.append(tok)
                if tok == self.image_token_id:
                    rows_e.append(feats[at:at + 1]); mask.append(True); at += 1
                else:
                    rows_e.append(zero(1)); mask.append(False)
            assert at == feats.shape[0]
        if next(it, None) is not None:
            raise ValueError("more images than image tokens")
        return ids, torch.cat(rows_e, 0), torch.tensor(mask, dtype=torch.bool, device=self.device)
