"""Vision service: CLIP image / text embeddings and their similarity (zero-shot scoring), SigLIP and
DINOv2 image embeddings.

Reference: src/HartsyInference.Engine/Services/VisionService.cs (embed operation),
src/HartsyInference.Vision/Embeddings/.
"""
from __future__ import annotations

import json
import threading
from pathlib import Path

import torch

from ..assets.safetensors import ShardedCheckpoint
from ..models.encoders.clip_vision import ClipVisionEncoder, clip_vision_from_hf, preprocess_image
from .requests import ModelSpec, VisionRequest, VisionResult


class _ClipDual:
    """Both towers of a Hugging Face ``CLIPModel`` checkpoint with their projections."""

    def __init__(self, path: str, device):
        from ..assets.tokenizer import ClipTokenizer
        from ..models.encoders.clip import ClipTextConfig, ClipTextEncoder
        p = Path(path)
        raw = json.loads((p / "config.json").read_text())
        ck = ShardedCheckpoint(p)
        self.device = torch.device(device)
        self.vision = ClipVisionEncoder(clip_vision_from_hf(raw["vision_config"]), device, get=ck.get, prefix="vision_model.")
        self.visual_proj = ck.get("visual_projection.weight").float().to(self.device)
        self.text = None
        tc = raw.get("text_config")
        has_tok = (p / "vocab.json").exists() or (p / "tokenizer.json").exists()
        if tc and has_tok and ck.get("text_projection.weight") is not None:
            width = tc.get("hidden_size", 512)
            cfg = ClipTextConfig(vocab_size=tc.get("vocab_size", 49408), width=width,
                                 layers=tc.get("num_hidden_layers", 12), heads=tc.get("num_attention_heads", 8),
                                 max_len=tc.get("max_position_embeddings", 77),
                                 mlp_ratio=tc.get("intermediate_size", 4 * width) // width,
                                 quick_gelu=tc.get("hidden_act", "quick_gelu") == "quick_gelu")
            self.text = ClipTextEncoder(cfg, device, get=ck.get)
            self.text_proj = ck.get("text_projection.weight").float().to(self.device)
            self.tokenizer = ClipTokenizer.from_dir(p, cfg.max_len)

    @staticmethod
    def _unit(x: torch.Tensor) -> torch.Tensor:
        return x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)

    def embed_images(self, images: list) -> torch.Tensor:
        size = self.vision.cfg.image_size
        feats = [self.vision.embed(preprocess_image(im, size)).float() @ self.visual_proj.t() for im in images]
        return self._unit(torch.stack(feats)).cpu()

    def embed_texts(self, texts: list[str]) -> torch.Tensor:
        if self.text is None:
            raise ValueError("this checkpoint has no text tower")
        feats = []
        for t in texts:
            _, pooled = self.text.encode(torch.tensor(self.tokenizer.encode(t)))
            feats.append(pooled.float() @ self.text_proj.t())
        return self._unit(torch.stack(feats)).cpu()


class _VitEmbedder:
    """A single-tower image embedder: SigLIP vision model or DINOv2."""
    SIGLIP_MEAN_STD = ((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))
    IMAGENET_MEAN_STD = ((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))

    def __init__(self, path: str, raw: dict, device):
        from ..models.encoders.vit import VitEncoder, vit_from_hf
        vc = raw.get("vision_config", raw)
        vc = {**vc, "model_type": "dinov2" if raw.get("model_type") == "dinov2" else "siglip"}
        ck = ShardedCheckpoint(path)
        self.enc = VitEncoder(vit_from_hf(vc), device, get=ck.get)
        self.mean, self.std = self.IMAGENET_MEAN_STD if vc["model_type"] == "dinov2" else self.SIGLIP_MEAN_STD

    def embed_images(self, images: list) -> torch.Tensor:
        from ..models.encoders.clip_vision import CLIP_MEAN, CLIP_STD
        size = self.enc.cfg.image_size
        cm, cs = torch.tensor(CLIP_MEAN)[:, None, None], torch.tensor(CLIP_STD)[:, None, None]
        m, sd = torch.tensor(self.mean)[:, None, None], torch.tensor(self.std)[:, None, None]
        feats = []
        for im in images:
            x = preprocess_image(im, size) * cs + cm           # back to [0, 1], then this family's statistics
            feats.append(self.enc.embed((x - m) / sd).float())
        return _ClipDual._unit(torch.stack(feats)).cpu()

    def embed_texts(self, texts):
        raise ValueError("this checkpoint embeds images only")


class _DepthEstimator:
    def __init__(self, path: str, raw: dict, device):
        from ..models.vision.depth_anything import DepthAnything, depth_anything_from_hf
        self.model = DepthAnything(depth_anything_from_hf(raw), device, get=ShardedCheckpoint(path).get)

    def depth(self, images: list, short_side: int = 518) -> list:
        import numpy as np
        P = self.model.cfg.backbone.patch
        mean = torch.tensor(_VitEmbedder.IMAGENET_MEAN_STD[0])[:, None, None]
        std = torch.tensor(_VitEmbedder.IMAGENET_MEAN_STD[1])[:, None, None]
        out = []
        for im in images:
            if isinstance(im, (str, bytes)) or hasattr(im, "__fspath__"):
                from PIL import Image
                im = Image.open(im)
            if hasattr(im, "convert"):
                im = torch.from_numpy(np.asarray(im.convert("RGB")).copy())
            t = torch.as_tensor(im)
            if t.dtype == torch.uint8:
                t = t.float() / 255.0
            if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
                t = t.permute(2, 0, 1)
            _, h, w = t.shape
            s = short_side / min(h, w)
            nh, nw = max(P, round(h * s / P) * P), max(P, round(w * s / P) * P)      # both sides multiples of the patch
            x = torch.nn.functional.interpolate(t.float()[None], size=(nh, nw), mode="bicubic", align_corners=False)[0].clamp(0, 1)
            d = self.model.predict((x - mean) / std)
            out.append(torch.nn.functional.interpolate(d[None, None].float().cpu(), size=(h, w), mode="bilinear", align_corners=False)[0, 0])
        return out


class _Segmenter:
    def __init__(self, path: str, raw: dict, device):
        from ..assets.tokenizer import ClipTokenizer
        from ..models.vision.clipseg import ClipSeg, clipseg_from_hf
        cfg = clipseg_from_hf(raw)
        self.model = ClipSeg(cfg, device, get=ShardedCheckpoint(path).get)
        self.tokenizer = ClipTokenizer.from_dir(path, cfg.text.max_len)

    def segment(self, images: list, texts: list[str]) -> list:
        size = self.model.cfg.vision.image_size
        conds = [self.model.text_embedding(torch.tensor(self.tokenizer.encode(t))) for t in texts]
        out = []
        for im in images:
            x = preprocess_image(im, size)
            h, w = _image_hw(im)
            maps = torch.stack([torch.sigmoid(self.model.segment(x, c)).float().cpu() for c in conds])
            out.append(torch.nn.functional.interpolate(maps[None], size=(h, w), mode="bilinear", align_corners=False)[0])
        return out


class _PromptSegmenter:
    """SAM 2: one mask per prompt (points and / or a box); of the three candidate masks the one with the
    highest predicted IoU is returned, as probabilities at the image's own size."""
    MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)

    def __init__(self, path: str, raw: dict, device):
        from ..models.vision.sam2 import Sam2, sam2_from_hf
        self.cfg = sam2_from_hf(raw)
        self.model = Sam2(self.cfg, device, get=ShardedCheckpoint(path).get)

    def segment(self, images: list, points: list, labels: list, boxes: list) -> tuple[list, list]:
        size = self.cfg.image_size
        n = max(len(points), len(boxes))
        if n == 0:
            raise ValueError("promptable segmentation needs points or boxes")
        if points and boxes and len(points) != len(boxes):
            raise ValueError("give as many boxes as point prompts (or only one of the two)")
        masks, scores = [], []
        for im in images:
            h, w = _image_hw(im)
            x = _Detector._squeeze(im, size)
            x = (x - torch.tensor(self.MEAN)[:, None, None]) / torch.tensor(self.STD)[:, None, None]
            sx, sy = size / w, size / h
            pts = lab = bxs = None
            if points:
                m = max(len(p) for p in points)
                pts = torch.zeros(1, n, m, 2)
                lab = torch.full((1, n, m), -10, dtype=torch.int64)           # padding points are ignored
                for i, p in enumerate(points):
                    for j, (px, py) in enumerate(p):
                        pts[0, i, j] = torch.tensor([px * sx, py * sy])
                        lab[0, i, j] = int(labels[i][j]) if (i < len(labels) and j < len(labels[i])) else 1
            if boxes:
                bxs = torch.tensor([[b[0] * sx, b[1] * sy, b[2] * sx, b[3] * sy] for b in boxes])[None]
            logits, iou, _ = self.model.segment(x[None], pts, lab, bxs, multimask=True)
            best = iou[0].argmax(-1)                                           # [n]
            pick = logits[0][torch.arange(n), best]                            # [n, h', w']
            up = torch.nn.functional.interpolate(pick[None].float().cpu(), size=(h, w), mode="bilinear", align_corners=False)[0]
            masks.append(torch.sigmoid(up))
            scores.append(iou[0][torch.arange(n), best].float().cpu())
        return masks, scores


def nms(boxes: torch.Tensor, scores: torch.Tensor, iou: float) -> list[int]:
    """Greedy non-maximum suppression over [n, 4] corner boxes; returns kept indices, best first."""
    order = scores.argsort(descending=True).tolist()
    keep: list[int] = []
    area = (boxes[:, 2] - boxes[:, 0]).clamp_min(0) * (boxes[:, 3] - boxes[:, 1]).clamp_min(0)
    while order:
        i = order.pop(0)
        keep.append(i)
        rest = []
        for j in order:
            w = (torch.minimum(boxes[i, 2], boxes[j, 2]) - torch.maximum(boxes[i, 0], boxes[j, 0])).clamp_min(0)
            h = (torch.minimum(boxes[i, 3], boxes[j, 3]) - torch.maximum(boxes[i, 1], boxes[j, 1])).clamp_min(0)
            inter = w * h
            if float(inter / (area[i] + area[j] - inter).clamp_min(1e-12)) <= iou:
                rest.append(j)
        order = rest
    return keep


class _Detector:
    def __init__(self, path: str, raw: dict, device):
        from ..assets.tokenizer import ClipTokenizer
        from ..models.vision.owlvit import OwlVit, owlvit_from_hf
        cfg = owlvit_from_hf(raw)
        self.model = OwlVit(cfg, device, get=ShardedCheckpoint(path).get)
        self.tokenizer = ClipTokenizer.from_dir(path, cfg.text.max_len)

    def detect(self, images: list, texts: list[str], threshold: float, iou: float) -> list:
        size = self.model.cfg.vision.image_size
        queries = torch.stack([self.model.text_embedding(torch.tensor(self.tokenizer.encode(t))) for t in texts])
        out = []
        for im in images:
            h, w = _image_hw(im)
            # the detector sees the whole picture squeezed to its input size; boxes scale back per axis
            x = preprocess_image(self._squeeze(im, size), size)
            logits, boxes = self.model.detect(x, queries)
            scores = torch.sigmoid(logits).float().cpu()
            b = boxes.float().cpu()
            corners = torch.stack([(b[:, 0] - b[:, 2] / 2) * w, (b[:, 1] - b[:, 3] / 2) * h,
                                   (b[:, 0] + b[:, 2] / 2) * w, (b[:, 1] + b[:, 3] / 2) * h], 1)
            found = []
            for qi, label in enumerate(texts):
                sel = (scores[:, qi] >= threshold).nonzero().flatten()
                for k in nms(corners[sel], scores[sel, qi], iou):
                    i = int(sel[k])
                    found.append({"label": label, "score": float(scores[i, qi]), "box": [float(v) for v in corners[i]]})
            out.append(sorted(found, key=lambda d: -d["score"]))
        return out

    @staticmethod
    def _squeeze(image, size: int) -> torch.Tensor:
        import numpy as np
        if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
            from PIL import Image
            image = Image.open(image)
        if hasattr(image, "convert"):
            image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
        t = torch.as_tensor(image)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
            t = t.permute(2, 0, 1)
        return torch.nn.functional.interpolate(t.float()[None], size=(size, size), mode="bicubic", align_corners=False,
                                               antialias=True)[0].clamp(0, 1)


class _SceneParser:
    """UperNet: a class per pixel (ADE20K-style label sets from the checkpoint's ``id2label``)."""

    MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)

    def __init__(self, path: str, raw: dict, device):
        from ..models.vision.upernet import UperNet, UperNetConfig
        self.model = UperNet(UperNetConfig.from_hf(raw), ShardedCheckpoint(path).get, device,
                             torch.bfloat16 if str(device).startswith("cuda") else torch.float32)
        self.names = {int(k): str(v) for k, v in (raw.get("id2label") or {}).items()}
        self.short_side = int(raw.get("short_side", 512))

    def parse(self, images: list):
        mean, std = torch.tensor(self.MEAN)[:, None, None], torch.tensor(self.STD)[:, None, None]
        maps, names = [], []
        for im in images:
            x = _as_chw(im)
            h, w = x.shape[-2:]
            scale = self.short_side / min(h, w)
            nh, nw = max(32, int(round(h * scale / 32)) * 32), max(32, int(round(w * scale / 32)) * 32)
            y = torch.nn.functional.interpolate(x[None], size=(nh, nw), mode="bilinear", align_corners=False, antialias=scale < 1)[0]
            logits = self.model.logits(((y - mean) / std)[None])
            labels = torch.nn.functional.interpolate(logits, size=(h, w), mode="bilinear", align_corners=False)[0].argmax(0).cpu()
            maps.append(labels)
            names.append([self.names.get(int(i), str(int(i))) for i in labels.unique()])
        return maps, names


class _GroundedDetector:
    """Grounding DINO: the queries are joined into one caption ("a cat . a remote control .") and every detection is
    labelled with the phrase whose tokens it matched best."""

    MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)

    def __init__(self, path: str, raw: dict, device):
        from ..assets.tokenizer import WordPieceTokenizer
        from ..models.vision.grounding_dino import GroundingDino, GroundingDinoConfig
        self.model = GroundingDino(GroundingDinoConfig.from_hf(raw), ShardedCheckpoint(path).get, device,
                                   torch.bfloat16 if str(device).startswith("cuda") else torch.float32)
        self.tokenizer = WordPieceTokenizer.from_dir(path)
        self.short_side = int(raw.get("short_side", 800))

    def detect(self, images: list, texts: list[str], threshold: float, iou: float) -> list:
        tok = self.tokenizer
        ids, spans = [tok.cls_id], []
        dot = tok.encode(".", add_special=False)
        for t in texts:
            piece = tok.encode(t.strip().lower().rstrip("."), add_special=False)
            spans.append((len(ids), len(ids) + len(piece)))
            ids += piece + dot
        ids.append(tok.sep_id)
        ids_t = torch.tensor(ids)
        mean, std = torch.tensor(self.MEAN)[:, None, None], torch.tensor(self.STD)[:, None, None]
        out = []
        for im in images:
            x = _as_chw(im)
            h, w = x.shape[-2:]
            scale = min(self.short_side / min(h, w), 1333 / max(h, w))
            nh, nw = max(32, int(round(h * scale))), max(32, int(round(w * scale)))
            x = torch.nn.functional.interpolate(x[None], size=(nh, nw), mode="bilinear", align_corners=False, antialias=scale < 1)[0]
            logits, boxes = self.model.forward(((x - mean) / std)[None], ids_t)
            probs = logits.sigmoid().cpu()
            boxes = boxes.cpu()
            per_phrase = torch.stack([probs[:, a:b].max(-1)[0] if b > a else torch.zeros(probs.shape[0]) for a, b in spans], 1)
            score, which = per_phrase.max(-1)
            corners = torch.stack([(boxes[:, 0] - boxes[:, 2] / 2) * w, (boxes[:, 1] - boxes[:, 3] / 2) * h,
                                   (boxes[:, 0] + boxes[:, 2] / 2) * w, (boxes[:, 1] + boxes[:, 3] / 2) * h], 1)
            found = []
            for qi, label in enumerate(texts):
                sel = ((which == qi) & (score >= threshold)).nonzero().flatten()
                for k in nms(corners[sel], score[sel], iou):
                    i = int(sel[k])
                    found.append({"label": label, "score": float(score[i]), "box": [float(v) for v in corners[i]]})
            out.append(sorted(found, key=lambda d_: -d_["score"]))
        return out


class _ClosedSetDetector:
    """RT-DETR: fixed label set from the checkpoint's ``id2label``; ``texts`` (optional) keep only the
    named labels."""

    def __init__(self, path: str, raw: dict, device):
        from ..models.vision.rtdetr import RtDetr, rtdetr_from_hf
        self.cfg = rtdetr_from_hf(raw)
        self.model = RtDetr(self.cfg, device, get=ShardedCheckpoint(path).get)

    def detect(self, images: list, texts: list, threshold: float, iou: float) -> list:
        size = self.cfg.image_size
        keep = {t.strip().lower() for t in (texts or [])}
        out = []
        for im in images:
            h, w = _image_hw(im)
            x = _Detector._squeeze(im, size)[None]                 # the whole picture squeezed to the input size, values in [0, 1]
            found = []
            for label, score, (cx, cy, bw, bh) in self.model.detect(x, threshold)[0]:
                name = self.cfg.id2label.get(label, str(label))
                if keep and name.lower() not in keep:
                    continue
                found.append({"label": name, "score": float(score),
                              "box": [(cx - bw / 2) * w, (cy - bh / 2) * h, (cx + bw / 2) * w, (cy + bh / 2) * h]})
            out.append(found)
        return out


COCO80 = ("person,bicycle,car,motorcycle,airplane,bus,train,truck,boat,traffic light,fire hydrant,stop sign,"
          "parking meter,bench,bird,cat,dog,horse,sheep,cow,elephant,bear,zebra,giraffe,backpack,umbrella,handbag,tie,"
          "suitcase,frisbee,skis,snowboard,sports ball,kite,baseball bat,baseball glove,skateboard,surfboard,"
          "tennis racket,bottle,wine glass,cup,fork,knife,spoon,bowl,banana,apple,sandwich,orange,broccoli,carrot,"
          "hot dog,pizza,donut,cake,chair,couch,potted plant,bed,dining table,toilet,tv,laptop,mouse,remote,keyboard,"
          "cell phone,microwave,oven,toaster,sink,refrigerator,book,clock,vase,scissors,teddy bear,hair drier,"
          "toothbrush")


def coco_names() -> list[str]:
    return COCO80.split(",")


class _YoloDetector:
    """YOLOv8 / YOLO11 (detect, segment, pose and face-landmark heads): a state dict (``.safetensors`` or ``.pt``) with the trainer's ``model.N.*`` names, BatchNorm folded
    or not. Labels come from ``names`` / ``id2label`` of a ``config.json`` beside it, else COCO's 80 when the head
    has 80 classes, else the class index."""

    def __init__(self, path: str, raw: dict, device):
        from ..models.vision.yolo import YoloV8, detect_size
        p = Path(path)
        if p.is_dir():
            files = sorted(p.glob("*.safetensors")) + sorted(p.glob("*.pt")) + sorted(p.glob("*.pth"))
            if not files:
                raise ValueError(f"{path}: no .safetensors or .pt file")
            p = files[0]
        if p.suffix == ".safetensors":
            from ..assets.safetensors import SafeTensorsFile
            f = SafeTensorsFile(p)
            tensors = {k: f.get(k) for k in f.keys()}
        else:
            from ..assets.torch_checkpoint import load_torch_checkpoint
            tensors = load_torch_checkpoint(p)
        self.cfg = detect_size(tensors.get)
        self.model = YoloV8(self.cfg, device, get=tensors.get)
        names = raw.get("names") or raw.get("id2label") or {}
        if isinstance(names, list):
            names = dict(enumerate(names))
        self.names = {int(k): str(v) for k, v in names.items()}
        if not self.names and self.cfg.num_classes == 80:
            self.names = dict(enumerate(coco_names()))
        elif not self.names and self.cfg.num_classes == 1 and self.cfg.task == "pose":
            self.names = {0: "person" if self.cfg.keypoints == 17 else "face"}
        self.size = int(raw.get("image_size", 640))

    def detect(self, images: list, texts: list, threshold: float, iou: float) -> list:
        """Boxes in the pixels of each picture. Pose / face checkpoints add ``keypoints`` ([K][x, y(, visibility)]),
        segmentation checkpoints ``mask`` (bool tensor [H, W] of the picture)."""
        keep = {t.strip().lower() for t in (texts or [])}
        out = []
        for im in images:
            x, scale, (px, py) = letterbox(_as_chw(im), self.size)
            h, w = _image_hw(im)
            found = []
            for d in self.model.detect(x[None], threshold, iou, full=True)[0]:
                name = self.names.get(d["label"], str(d["label"]))
                if keep and name.lower() not in keep:
                    continue
                x0, y0, x1, y1 = d["box"]
                box = [(x0 - px) / scale, (y0 - py) / scale, (x1 - px) / scale, (y1 - py) / scale]
                item = {"label": name, "score": d["score"],
                        "box": [min(max(box[0], 0.0), w), min(max(box[1], 0.0), h), min(max(box[2], 0.0), w), min(max(box[3], 0.0), h)]}
                if "keypoints" in d:
                    k = d["keypoints"].clone()
                    k[:, 0], k[:, 1] = (k[:, 0] - px) / scale, (k[:, 1] - py) / scale
                    item["keypoints"] = k.tolist()
                if "mask" in d:
                    nh, nw = max(int(round(h * scale)), 1), max(int(round(w * scale)), 1)
                    m = d["mask"][py:py + nh, px:px + nw].float()[None, None]
                    item["mask"] = torch.nn.functional.interpolate(m, size=(h, w), mode="bilinear", align_corners=False)[0, 0] > 0.5
                found.append(item)
            out.append(found)
        return out


def _as_chw(image) -> torch.Tensor:
    import numpy as np
    if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
        from PIL import Image
        image = Image.open(image)
    if hasattr(image, "convert"):
        image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
    t = torch.as_tensor(image)
    if t.dtype == torch.uint8:
        t = t.float() / 255.0
    if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
        t = t.permute(2, 0, 1)
    return t.float()


def letterbox(chw: torch.Tensor, size: int, fill: float = 114 / 255):
    """Aspect-preserving resize of [3, H, W] into a ``size`` x ``size`` square, centred on grey. Returns the square,
    the scale applied and the (x, y) padding, so a box maps back as ``(v - pad) / scale``."""
    _, h, w = chw.shape
    scale = min(size / h, size / w)
    nh, nw = max(int(round(h * scale)), 1), max(int(round(w * scale)), 1)
    r = torch.nn.functional.interpolate(chw[None], size=(nh, nw), mode="bilinear", align_corners=False, antialias=scale < 1)[0]
    out = torch.full((3, size, size), fill)
    py, px = (size - nh) // 2, (size - nw) // 2
    out[:, py:py + nh, px:px + nw] = r.clamp(0, 1)
    return out, scale, (px, py)


def _image_hw(image) -> tuple[int, int]:
    if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
        from PIL import Image
        image = Image.open(image)
    if hasattr(image, "size") and hasattr(image, "convert"):
        return image.size[1], image.size[0]
    t = torch.as_tensor(image)
    return (t.shape[0], t.shape[1]) if (t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3) else (t.shape[-2], t.shape[-1])


class VisionService:
    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict[str, _ClipDual] = {}

    def loaded_keys(self) -> list[str]:
        return [f"clip:{k}" for k in self._loaded]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def _model(self, spec: ModelSpec) -> _ClipDual:
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._loaded:
                cfg_file = Path(path) / "config.json"
                raw = json.loads(cfg_file.read_text()) if cfg_file.is_file() else {}
                mt = raw.get("model_type", "clip" if raw else "yolov8")
                if str(mt).startswith("yolo"):
                    self._loaded[path] = _YoloDetector(path, raw, self.device)
                elif mt == "depth_anything":
                    self._loaded[path] = _DepthEstimator(path, raw, self.device)
                elif mt == "clipseg":
                    self._loaded[path] = _Segmenter(path, raw, self.device)
                elif mt in ("owlvit", "owlv2"):
                    self._loaded[path] = _Detector(path, raw, self.device)
                elif mt == "upernet":
                    self._loaded[path] = _SceneParser(path, raw, self.device)
                elif mt in ("grounding-dino", "grounding_dino", "mm-grounding-dino"):
                    self._loaded[path] = _GroundedDetector(path, raw, self.device)
                elif mt in ("sam2", "sam2_video"):
                    self._loaded[path] = _PromptSegmenter(path, raw, self.device)
                elif mt == "rt_detr":
                    self._loaded[path] = _ClosedSetDetector(path, raw, self.device)
                elif mt in ("siglip", "siglip_vision_model", "dinov2"):
                    self._loaded[path] = _VitEmbedder(path, raw, self.device)
                else:
                    self._loaded[path] = _ClipDual(path, self.device)
            return self._loaded[path]

    def _annotate(self, spec: ModelSpec, req: VisionRequest) -> VisionResult:
        from ..models.vision import annotators as A
        out = VisionResult(control_images=[])
        kind = req.annotator
        if kind in ("canny", "tile", "blur"):
            for im in req.images:
                x = _as_chw(im)
                if kind == "canny":
                    e = A.canny(x, req.canny_low, req.canny_high)
                    out.control_images.append((e[..., None].expand(-1, -1, 3) * 255).to(torch.uint8).contiguous())
                else:
                    y = A.pixelate(x) if kind == "tile" else A.tile_blur(x)
                    out.control_images.append((y.clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).contiguous())
            return out
        if kind not in ("pose", "depth", "segmentation"):
            raise ValueError(f"annotator '{kind}' is not built (canny, tile, blur, pose, depth and segmentation are)")
        m = self._model(spec)
        if kind == "pose":
            if not isinstance(m, _YoloDetector) or m.cfg.task != "pose":
                raise ValueError("the pose annotator needs a pose checkpoint")
            found = m.detect(req.images, [], req.score_threshold, req.nms_iou)
            for im, people in zip(req.images, found):
                h, w = _image_hw(im)
                out.control_images.append(A.render_pose([torch.tensor(p["keypoints"]) for p in people], h, w))
        elif kind == "depth":
            if not isinstance(m, _DepthEstimator):
                raise ValueError("the depth annotator needs a depth checkpoint")
            out.control_images = [A.depth_control(torch.as_tensor(d)) for d in m.depth(req.images, getattr(req, "short_side", 518))]
        elif kind == "segmentation":
            if not isinstance(m, _SceneParser):
                raise ValueError("the segmentation annotator needs a scene-parsing checkpoint")
            out.control_images = [A.label_palette(l) for l in m.parse(req.images)[0]]
        return out

    def run(self, spec: ModelSpec, req: VisionRequest) -> VisionResult:
        if req.operation == "annotate":
            return self._annotate(spec, req)
        if req.operation not in ("embed", "depth", "segment", "detect"):
            raise ValueError(f"vision operation '{req.operation}' is not built (embed, depth, segment, detect and annotate are)")
        m = self._model(spec)
        out = VisionResult()
        if req.operation == "detect":
            if isinstance(m, (_ClosedSetDetector, _YoloDetector)):
                out.detections = m.detect(req.images, req.texts, req.score_threshold, req.nms_iou)
                return out
            if not isinstance(m, (_Detector, _GroundedDetector)):
                raise ValueError("this checkpoint is not a detector")
            if not req.texts:
                raise ValueError("detect needs at least one text query")
            out.detections = m.detect(req.images, req.texts, req.score_threshold, req.nms_iou)
            return out
        if isinstance(m, (_Detector, _GroundedDetector, _ClosedSetDetector, _YoloDetector)):
            raise ValueError("this checkpoint detects; use operation 'detect'")
        if req.operation == "segment" and isinstance(m, _SceneParser):
            out.masks, out.labels = m.parse(req.images)
            return out
        if isinstance(m, _SceneParser):
            raise ValueError("this checkpoint labels every pixel; use operation 'segment'")
        if req.operation == "segment" and isinstance(m, _PromptSegmenter):
            out.masks, out.mask_scores = m.segment(req.images, req.points, req.point_labels, req.boxes)
            return out
        if isinstance(m, _PromptSegmenter):
            raise ValueError("this checkpoint segments from point / box prompts; use operation 'segment'")
        if req.operation == "segment":
            if not isinstance(m, _Segmenter):
                raise ValueError("this checkpoint is not a text-prompted segmenter")
            if not req.texts:
                raise ValueError("segment needs at least one text prompt")
            out.masks = m.segment(req.images, req.texts)
            return out
        if isinstance(m, _Segmenter):
            raise ValueError("this checkpoint segments; use operation 'segment'")
        if req.operation == "depth":
            if not isinstance(m, _DepthEstimator):
                raise ValueError("this checkpoint is not a depth estimator")
            out.depth = m.depth(req.images, getattr(req, "short_side", 518))
            return out
        if isinstance(m, _DepthEstimator):
            raise ValueError("this checkpoint estimates depth; use operation 'depth'")
        if req.images:
            out.image_embeddings = m.embed_images(req.images)
        if req.texts:
            out.text_embeddings = m.embed_texts(req.texts)
        if req.images and req.texts:
            out.similarity = out.image_embeddings @ out.text_embeddings.t()
        return out


class RestoreService:
    """Image restoration: Real-ESRGAN upscaling from a ``.safetensors`` / ``.pth`` file or a directory
    holding one. Reference: src/HartsyInference.Engine/Services/RestoreService.cs."""

    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict = {}

    def loaded_keys(self) -> list[str]:
        return [f"esrgan:{k}" for k in self._loaded]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def _net(self, spec: ModelSpec):
        from ..models.vision.rrdbnet import RrdbNet, detect_rrdb_config
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._loaded:
                p = Path(path)
                if p.is_dir():
                    files = sorted(p.glob("*.safetensors")) + sorted(p.glob("*.pth"))
                    if not files:
                        raise ValueError(f"{path}: no .safetensors or .pth file")
                    p = files[0]
                if p.suffix == ".safetensors":
                    from ..assets.safetensors import SafeTensorsFile
                    f = SafeTensorsFile(p)
                    tensors = {k: f.get(k) for k in f.keys()}
                else:
                    from ..assets.torch_checkpoint import load_torch_checkpoint
                    tensors = load_torch_checkpoint(p)
                dt = torch.bfloat16 if str(self.device).startswith("cuda") else torch.float32
                self._loaded[path] = RrdbNet(detect_rrdb_config(tensors.keys()), self.device, dt, get=tensors.get)
            return self._loaded[path]

    def run(self, spec: ModelSpec, req):
        from ..models.vision.rrdbnet import UpscalePipeline
        if req.operation != "upscale":
            raise ValueError(f"restore operation '{req.operation}' is not built (upscale is)")
        if req.image is None:
            raise ValueError("RestoreRequest.image is empty")
        img = req.image
        if not (isinstance(img, torch.Tensor) and img.is_floating_point()):
            import numpy as np
            if isinstance(img, (str, bytes)) or hasattr(img, "__fspath__"):
                from PIL import Image
                img = Image.open(img)
            if hasattr(img, "convert"):
                img = torch.from_numpy(np.asarray(img.convert("RGB")).copy())
            img = torch.as_tensor(img)
            if img.dtype == torch.uint8:
                img = img.float() / 255.0
            if img.ndim == 3 and img.shape[-1] == 3 and img.shape[0] != 3:
                img = img.permute(2, 0, 1)
        pipe = UpscalePipeline(self._net(spec), req.tile, req.tile_overlap)
        up = pipe.upscale_tensor(img.float().clamp(0, 1))
        from .requests import ImageResult
        u8 = (up * 255.0).round().to(torch.uint8).permute(1, 2, 0).contiguous()
        return ImageResult(rgb=u8.numpy().tobytes(), width=up.shape[2], height=up.shape[1], seed=0,
                           meta={"operation": "upscale", "scale": pipe.net.scale})
