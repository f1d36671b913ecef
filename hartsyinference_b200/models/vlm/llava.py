"""LLaVA-style vision-language model.

``<image>`` in the prompt expands to one placeholder token per image patch; the CLIP vision tower's
patch states (second-to-last layer, class token dropped) go through a two-layer GELU projector and
replace the embeddings of those placeholders. Everything after that is the ordinary decoder:
the serving engine prefills the mixed embeddings (``LLMEngine.add_request(..., prompt_embeds=...)``)
and decodes token by token with its paged KV cache.

Reference: src/HartsyInference.LLM/Multimodal/ (LLaVA-NeXT / Mllama / Qwen-VL generators,
MultimodalGenerator). Tensor names follow llava-hf checkpoints: ``vision_tower.vision_model.*``,
``multi_modal_projector.linear_1|2``, ``language_model.*``.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from ... import ops
from ..dit.common import WeightFactory
from ..encoders.clip_vision import ClipVisionConfig, ClipVisionEncoder
from ..llm.transformer import DecoderModel


class LlavaModel:
    def __init__(self, decoder: DecoderModel, vision_cfg: ClipVisionConfig, image_token_id: int,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0, feature_layer: int = -2):
        self.decoder = decoder
        self.device = decoder.device
        self.image_token_id = image_token_id
        self.feature_layer = feature_layer
        self.vision = ClipVisionEncoder(vision_cfg, self.device, get=get, seed=seed, prefix="vision_tower.vision_model.")
        f = WeightFactory(self.device, False, get=get, seed=seed + 1)
        H = decoder.cfg.hidden_size
        self.proj1 = f.linear("multi_modal_projector.linear_1", H, vision_cfg.width)
        self.proj2 = f.linear("multi_modal_projector.linear_2", H, H)

    @torch.no_grad()
    def image_features(self, image: torch.Tensor) -> torch.Tensor:
        """[num_patches, hidden] embeddings of one image in the decoder's space."""
        h = self.vision.hidden_states(image, self.feature_layer)[1:].contiguous()
        y = ops.linear(h, self.proj1).float()
        y = torch.nn.functional.gelu(y).to(torch.bfloat16)
        return ops.linear(y, self.proj2)

    def expand_prompt(self, token_ids: Sequence[int], images: Sequence[torch.Tensor]):
        """Replace every image token by ``num_patches`` placeholders. Returns (ids, embeds [T, H],
        mask [T]) where ``mask`` marks the rows whose embedding comes from an image."""
        return self._splice(token_ids, [self.image_features(im) for im in images])

    def _splice(self, token_ids: Sequence[int], feats: list):
        ids: list[int] = []
        rows: list[torch.Tensor] = []
        mask: list[bool] = []
        it = iter(feats)
        H = self.decoder.cfg.hidden_size
        for t in token_ids:
            if t == self.image_token_id:
                f = next(it, None)
                if f is None:
                    raise ValueError("more image tokens than images")
                ids += [self.image_token_id] * f.shape[0]
                rows.append(f)
                mask += [True] * f.shape[0]
            else:
                ids.append(int(t))
                rows.append(torch.zeros(1, H, dtype=torch.bfloat16, device=self.device))
                mask.append(False)
        if next(it, None) is not None:
            raise ValueError("more images than image tokens")
        return ids, torch.cat(rows, 0), torch.tensor(mask, dtype=torch.bool, device=self.device)

    def generate(self, engine, token_ids: Sequence[int], images: Sequence[torch.Tensor], params=None) -> list[int]:
        """Greedy / sampled generation through a serving engine built on ``self.decoder``."""
        ids, embeds, mask = self.expand_prompt(token_ids, images)
        rid = engine.add_request(ids, params, prompt_embeds=embeds, embeds_mask=mask)
        engine.run_until_done()
        return engine.requests[rid].output
