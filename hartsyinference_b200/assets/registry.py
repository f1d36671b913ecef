"""Model family detection from tensor names and metadata.

A checkpoint is classified without loading tensor data: GGUF files by ``general.architecture``,
Hugging Face directories by ``config.json``'s ``model_type``, bare safetensors files by marker
tensor names. Reference: src/HartsyInference.ModelAssets/Registry/ModelArchitectureDetector.cs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable


@dataclass(frozen=True)
class Detected:
    family: str            # "llm" | "dit-image" | "dit-video" | "vae" | "text-encoder" | "lora" | "unknown"
    arch: str              # e.g. "llama", "deepseek3", "flux", "wan", "t5", "clip", "sdxl"
    detail: str = ""


_MARKERS: list[tuple[str, str, tuple[str, ...]]] = [
    ("lora", "lora", ("lora_A.", "lora_down.", "lora.down.")),
    ("dit-image", "flux", ("double_blocks.0.img_attn.qkv.weight", "single_blocks.0.linear1.weight",
                           "transformer_blocks.0.attn.add_q_proj.weight")),
    ("dit-video", "wan", ("blocks.0.cross_attn.k.weight", "blocks.0.self_attn.norm_q.weight",
                          "patch_embedding.weight")),
    ("dit-image", "sd3", ("joint_blocks.0.x_block.attn.qkv.weight",)),
    ("dit-image", "sdxl", ("conditioner.embedders.1.model.ln_final.weight", "down_blocks.2.attentions.1.transformer_blocks.9.attn1.to_q.weight")),
    ("dit-image", "sd15", ("model.diffusion_model.input_blocks.0.0.weight",)),
    ("vae", "vae3d", ("decoder.conv1.weight", "decoder.middle.0.residual.0.gamma")),
    ("vae", "vae2d", ("decoder.mid_block.attentions.0.to_q.weight", "decoder.mid.attn_1.q.weight", "decoder.conv_in.weight")),
    ("text-encoder", "t5", ("encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight",)),
    ("text-encoder", "clip", ("text_model.encoder.layers.0.self_attn.q_proj.weight",)),
    ("llm", "deepseek3", ("model.layers.0.self_attn.kv_a_proj_with_mqa.weight",)),
    ("llm", "mixtral", ("model.layers.0.block_sparse_moe.gate.weight",)),
    ("llm", "moe", ("model.layers.0.mlp.experts.0.gate_proj.weight", "model.layers.1.mlp.experts.0.gate_proj.weight")),
    ("llm", "mamba", ("backbone.layers.0.mixer.A_log",)),
    ("llm", "bert", ("encoder.layer.0.attention.self.query.weight", "bert.encoder.layer.0.attention.self.query.weight")),
    ("llm", "llama", ("model.layers.0.self_attn.q_proj.weight",)),
    ("llm", "gpt2", ("h.0.attn.c_attn.weight", "transformer.h.0.attn.c_attn.weight")),
]


def detect_from_keys(keys: Iterable[str]) -> Detected:
    names = list(keys)
    joined = set(names)
    for family, arch, markers in _MARKERS:
        for mk in markers:
            if mk in joined or any(mk in n for n in names):
                return Detected(family, arch, f"marker '{mk}'")
    return Detected("unknown", "unknown")


def detect(path: str | Path) -> Detected:
    """Classify a file or directory."""
    p = Path(path)
    if p.is_dir():
        cfg = p / "config.json"
        if cfg.exists():
            d = json.loads(cfg.read_text())
            mt = d.get("model_type") or (d.get("_class_name") or "").lower()
            if mt:
                fam = "llm"
                if "flux" in mt:
                    fam = "dit-image"
                elif "wan" in mt:
                    fam = "dit-video"
                elif mt in ("t5", "umt5", "clip_text_model", "clip"):
                    fam = "text-encoder"
                elif "autoencoder" in mt:
                    fam = "vae"
                return Detected(fam, mt, "config.json")
        files = sorted(p.glob("*.safetensors")) + sorted(p.glob("*.gguf"))
        if not files:
            return Detected("unknown", "unknown", "empty directory")
        p = files[0]
    if p.suffix == ".gguf":
        from .gguf import GgufFile
        g = GgufFile(p)
        try:
            arch = str(g.metadata.get("general.architecture", "unknown"))
            names = g.keys()
        finally:
            g.close()
        if arch in ("flux", "wan", "sd3"):
            return Detected("dit-video" if arch == "wan" else "dit-image", arch, "gguf metadata")
        if arch == "unknown":
            return detect_from_keys(names)
        return Detected("llm", arch, "gguf metadata")
    if p.suffix == ".safetensors":
        from .safetensors import SafeTensorsFile
        f = SafeTensorsFile(p)
        try:
            return detect_from_keys(f.keys())
        finally:
            f.close()
    return Detected("unknown", "unknown", f"unsupported file type {p.suffix}")
