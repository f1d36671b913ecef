"""X-Codec: a speech / music codec whose tokens carry semantic content as well as acoustics (the codec
behind YuE-class music language models).

encode: the waveform goes two ways. (a) acoustic: the DAC encoder (total stride = the hop); (b)
semantic: a HuBERT-class model run on the waveform padded by half a hop on both sides, its
``layers + 1`` hidden states averaged, then a small convolutional encoder (a 3-tap convolution and
residual-unit blocks with strided convolutions) brings them to the acoustic frame rate. Both are
concatenated on the channel axis, mixed by a linear layer and quantised by a residual chain of
Euclidean codebooks. decode: the summed codebook vectors go through a linear layer to the DAC
decoder (without its final tanh; odd strides emit one extra sample).

Weights by the names of the `transformers` checkpoint (``acoustic_encoder.*``, ``acoustic_decoder.*``,
``semantic_model.*``, ``encoder_semantic.*``, ``fc``, ``fc2``, ``quantizer.quantizers.N.codebook.embed``).
Reference: src/HartsyInference.Audio/Models/Codecs/XCodec/.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .dac import DacCodec, DacConfig
from .hubert import Hubert, HubertConfig


class XCodec:
    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu"):
        self.device = torch.device(device)
        self._get, self._cache = get, {}
        ac = raw.get("acoustic_model_config", {})
        self.dac_cfg = DacConfig.from_hf(ac)
        rename = lambda n: ("acoustic_" + n) if n.startswith(("encoder.", "decoder.")) else n
        self.dac = DacCodec(self.dac_cfg, lambda n: get(rename(n)), device, final_tanh=False, odd_stride_padding=True)
        self.semantic = Hubert(HubertConfig.from_hf(raw.get("semantic_model_config", {})), lambda n: get("semantic_model." + n), device)
        self.hop = raw.get("hop_length") or self.dac_cfg.hop
        self.pad = self.hop // 2
        self.strides = tuple(raw.get("strides", (1, 1)))
        self.dilations = tuple(raw.get("block_dilations", (1, 1)))
        self.unit_kernel = raw.get("unit_kernel_size", 3)
        self.kernel = raw.get("kernel_size", 3)
        self.quantizers = raw.get("num_quantizers", 8)
        self.codebook_size = raw.get("codebook_size", 1024)
        self.sampling_rate = raw.get("sample_rate", raw.get("sampling_rate", 16000))

    def _w(self, name: str, optional: bool = False):
        hit = self._cache.get(name, False)
        if hit is False:
            t = self._get(name)
            if t is None and not optional:
                raise KeyError(name)
            hit = None if t is None else t.float().to(self.device)
            self._cache[name] = hit
        return hit

    def _semantic_frames(self, wave: torch.Tensor) -> torch.Tensor:
        """wave [B, samples] -> [B, C, frames] at the acoustic frame rate."""
        states = self.semantic.all_hidden_states(F.pad(wave, (self.pad, self.pad)))
        x = torch.stack(states, 1).mean(1).float().transpose(1, 2)
        x = F.conv1d(x, self._w("encoder_semantic.conv.weight"), padding=self.kernel // 2)
        for i, stride in enumerate(self.strides):
            p = f"encoder_semantic.conv_blocks.{i}"
            for j, dil in enumerate(self.dilations):
                y = F.conv1d(F.elu(x), self._w(f"{p}.res_units.{j}.conv1.weight"), dilation=dil, padding=((self.unit_kernel - 1) // 2) * dil)
                x = x + F.conv1d(F.elu(y), self._w(f"{p}.res_units.{j}.conv2.weight"))
            k = 3 if stride == 1 else 2 * stride
            x = F.conv1d(x, self._w(p + ".conv.weight"), self._w(p + ".conv.bias"), stride=stride, padding=(k - 1) // 2)
        return x

    def _book(self, i: int) -> torch.Tensor:
        return self._w(f"quantizer.quantizers.{i}.codebook.embed")

    @torch.no_grad()
    def encode(self, wave: torch.Tensor, quantizers: Optional[int] = None) -> torch.Tensor:
        """wave [B, samples] (or [B, 1, samples]) -> codes [B, n, frames]."""
        x = wave.to(self.device).float()
        x = x[:, 0] if x.dim() == 3 else x
        sem = self._semantic_frames(x)
        acoustic = self.dac.encode_latents(x, pad_to_hop=False)
        if acoustic.shape[-1] != sem.shape[-1]:
            acoustic = self.dac.encode_latents(F.pad(x, (self.pad, self.pad)), pad_to_hop=False)
        z = F.linear(torch.cat([acoustic, sem], 1).transpose(1, 2), self._w("fc.weight"), self._w("fc.bias"))      # [B, T, C]
        codes, residual = [], z
        for i in range(quantizers or self.quantizers):
            book = self._book(i)
            dist = residual.pow(2).sum(-1, keepdim=True) - 2 * residual @ book.t() + book.pow(2).sum(-1)[None, None]
            idx = dist.argmin(-1)
            residual = residual - book[idx]
            codes.append(idx)
        return torch.stack(codes, 1)

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> wave [B, samples]."""
        codes = codes.to(self.device).long().clamp(0, self.codebook_size - 1)
        q = sum(self._book(i)[codes[:, i]] for i in range(codes.shape[1]))                                          # [B, T, C]
        z = F.linear(q, self._w("fc2.weight"), self._w("fc2.bias")).transpose(1, 2)
        return self.dac.decode_latents(z)
