"""OWL-ViT open-vocabulary object detection.

Every image patch is a detection candidate: the CLIP vision tower's patch tokens (after the final
LayerNorm) are multiplied by the class token, normalised, and fed to two heads. The class head
projects a patch into the text embedding space and scores it against each text query by cosine
similarity with a learned per-patch shift and scale; the box head is a three-layer MLP whose output
is added to a bias that places each box at its patch's position with the patch's size, then squashed
to (cx, cy, w, h) in [0, 1].

Reference: src/HartsyInference.Vision/Detection/ (open-vocabulary detector behind the vision
service's detect operation). Tensor names follow Hugging Face ``OwlViTForObjectDetection``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..encoders.clip import ClipTextConfig, ClipTextEncoder, clip_text_from_hf
from ..encoders.clip_vision import ClipVisionConfig, ClipVisionEncoder, clip_vision_from_hf


@dataclass(frozen=True)
class OwlVitConfig:
    vision: ClipVisionConfig
    text: ClipTextConfig
    projection_dim: int = 512


def owlvit_from_hf(d: dict) -> OwlVitConfig:
    return OwlVitConfig(clip_vision_from_hf(d["vision_config"]), clip_text_from_hf(d["text_config"]), d.get("projection_dim", 512))


class OwlVit:
    def __init__(self, cfg: OwlVitConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        sub = None if get is None else (lambda n: get("owlvit." + n))
        self.vision = ClipVisionEncoder(cfg.vision, device, get=sub, seed=seed, prefix="vision_model.", pre_ln="pre_layernorm")
        self.text = ClipTextEncoder(cfg.text, device, get=sub, seed=seed + 1)
        self._get, self._g = get, torch.Generator().manual_seed(seed + 2)
        self.w: dict[str, torch.Tensor] = {}
        if get is None:
            self.text.projection = torch.randn(cfg.projection_dim, cfg.text.width, generator=self._g).to(self.device) * 0.05

    def _p(self, name: str, *shape, ones: bool = False) -> torch.Tensor:
        t = self.w.get(name)
        if t is None:
            t = self._get(name) if self._get is not None else None
            if t is None:
                if self._get is not None:
                    raise KeyError(name)
                fan = shape[-1] if len(shape) > 1 else 1
                t = torch.ones(*shape) if ones else torch.zeros(*shape) if name.endswith("bias") else \
                    torch.randn(*shape, generator=self._g) * (1.0 / fan) ** 0.5
            t = t.float().to(self.device)
            self.w[name] = t
        return t

    def _lin(self, x, name, o, i):
        return F.linear(x, self._p(name + ".weight", o, i), self._p(name + ".bias", o))

    @torch.no_grad()
    def text_embedding(self, ids: torch.Tensor) -> torch.Tensor:
        return self.text.encode(ids, project=True)[1].float()

    @staticmethod
    def box_bias(gh: int, gw: int) -> torch.Tensor:
        """[gh * gw, 4] logits that, alone, put a box of one patch's size on each patch's far corner."""
        xs = torch.arange(1, gw + 1, dtype=torch.float32) / gw
        ys = torch.arange(1, gh + 1, dtype=torch.float32) / gh
        yy, xx = torch.meshgrid(ys, xs, indexing="ij")
        xy = torch.stack([xx, yy], -1).reshape(-1, 2).clamp(0, 1)
        size = torch.tensor([1.0 / gw, 1.0 / gh]).expand_as(xy)
        logit = lambda t: torch.log(t + 1e-4) - torch.log1p(-t + 1e-4)
        return torch.cat([logit(xy), logit(size)], -1)

    @torch.no_grad()
    def detect(self, image: torch.Tensor, queries: torch.Tensor):
        """image [3, S, S] normalised (CLIP statistics), queries [Q, projection_dim] ->
        (logits [patches, Q], boxes [patches, 4] as normalised cx, cy, w, h)."""
        cfg = self.cfg
        W, Tw = cfg.vision.width, cfg.text.width
        x = self.vision.hidden_states(image).float()
        x = F.layer_norm(x, (W,), self.vision.post_w.float(), self.vision.post_b.float(), cfg.vision.eps)
        feats = F.layer_norm(x[1:] * x[:1], (W,), self._p("layer_norm.weight", W, ones=True), self._p("layer_norm.bias", W), 1e-5)
        cls = self._lin(feats, "class_head.dense0", Tw, W)        # the text width equals the projection width in these models
        cls = cls / (cls.norm(dim=-1, keepdim=True) + 1e-6)
        q = queries.to(self.device).float()
        q = q / (q.norm(dim=-1, keepdim=True) + 1e-6)
        shift = self._lin(feats, "class_head.logit_shift", 1, W)
        scale = F.elu(self._lin(feats, "class_head.logit_scale", 1, W)) + 1
        logits = (cls @ q.t() + shift) * scale
        h = F.gelu(self._lin(feats, "box_head.dense0", W, W))
        h = F.gelu(self._lin(h, "box_head.dense1", W, W))
        g = int(round(feats.shape[0] ** 0.5))
        boxes = torch.sigmoid(self._lin(h, "box_head.dense2", 4, W) + self.box_bias(g, g).to(self.device))
        return logits, boxes
