"""VITS text-to-speech (the architecture of MMS-TTS and Piper voices), inference path.

text ids -> text encoder (self-attention with learned relative-position keys / values inside a
window, convolutional feed-forward, post-LayerNorm) -> per-token prior mean / log-variance and a
duration (stochastic predictor: a spline-flow run in reverse from noise, or the plain convolutional
predictor) -> the prior is repeated per frame, sampled, and pushed backwards through the residual
coupling flow (WaveNet-conditioned mean shifts) -> HiFi-GAN turns the latent frames into a waveform.

One utterance at a time, so there is no padding mask. The 1-D convolutions go through PyTorch
(they are off the named hot paths); with both noise scales at zero the output is deterministic.

Reference: src/HartsyInference.Audio/Models/Vits/, src/HartsyInference.Audio/Pipelines/PiperPipeline.cs,
src/HartsyInference.Audio/Models/Vocoders/ (HiFi-GAN). Tensor names follow Hugging Face ``VitsModel``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class VitsConfig:
    vocab_size: int = 38
    hidden: int = 192
    layers: int = 6
    heads: int = 2
    window: int = 4
    ffn: int = 768
    ffn_kernel: int = 3
    flow_size: int = 192
    spectrogram_bins: int = 513
    eps: float = 1e-5
    stochastic_duration: bool = True
    dp_kernel: int = 3
    dp_filter: int = 256
    dp_flows: int = 4
    dp_bins: int = 10
    dp_tail_bound: float = 5.0
    dds_layers: int = 3
    dds_kernel: int = 3
    prior_flows: int = 4
    wavenet_layers: int = 4
    wavenet_kernel: int = 5
    wavenet_dilation: int = 1
    upsample_initial: int = 512
    upsample_rates: tuple = (8, 8, 2, 2)
    upsample_kernels: tuple = (16, 16, 4, 4)
    resblock_kernels: tuple = (3, 7, 11)
    resblock_dilations: tuple = ((1, 3, 5), (1, 3, 5), (1, 3, 5))
    leaky_slope: float = 0.1
    num_speakers: int = 1
    speaker_dim: int = 0
    sampling_rate: int = 16000
    noise_scale: float = 0.667
    noise_scale_duration: float = 0.8
    speaking_rate: float = 1.0

    @property
    def hop(self) -> int:
        out = 1
        for r in self.upsample_rates:
            out *= r
        return out


def tiny_vits(**over) -> VitsConfig:
    base = dict(vocab_size=40, hidden=64, layers=2, heads=2, ffn=128, flow_size=64, spectrogram_bins=33, upsample_initial=64,
                upsample_rates=(4, 4), upsample_kernels=(8, 8), resblock_kernels=(3, 5), resblock_dilations=((1, 3), (1, 3)),
                prior_flows=2, wavenet_layers=2, dp_flows=2, dp_filter=32, dds_layers=2)
    base.update(over)
    return VitsConfig(**base)


def vits_from_hf(d: dict) -> VitsConfig:
    return VitsConfig(
        vocab_size=d["vocab_size"], hidden=d["hidden_size"], layers=d["num_hidden_layers"], heads=d["num_attention_heads"],
        window=d.get("window_size", 4), ffn=d["ffn_dim"], ffn_kernel=d.get("ffn_kernel_size", 3), flow_size=d["flow_size"],
        spectrogram_bins=d.get("spectrogram_bins", 513), eps=d.get("layer_norm_eps", 1e-5),
        stochastic_duration=bool(d.get("use_stochastic_duration_prediction", True)),
        dp_kernel=d.get("duration_predictor_kernel_size", 3), dp_filter=d.get("duration_predictor_filter_channels", 256),
        dp_flows=d.get("duration_predictor_num_flows", 4), dp_bins=d.get("duration_predictor_flow_bins", 10),
        dp_tail_bound=d.get("duration_predictor_tail_bound", 5.0), dds_layers=d.get("depth_separable_num_layers", 3),
        dds_kernel=d.get("duration_predictor_kernel_size", 3), prior_flows=d.get("prior_encoder_num_flows", 4),
        wavenet_layers=d.get("prior_encoder_num_wavenet_layers", 4), wavenet_kernel=d.get("wavenet_kernel_size", 5),
        wavenet_dilation=d.get("wavenet_dilation_rate", 1), upsample_initial=d.get("upsample_initial_channel", 512),
        upsample_rates=tuple(d.get("upsample_rates", (8, 8, 2, 2))), upsample_kernels=tuple(d.get("upsample_kernel_sizes", (16, 16, 4, 4))),
        resblock_kernels=tuple(d.get("resblock_kernel_sizes", (3, 7, 11))),
        resblock_dilations=tuple(tuple(x) for x in d.get("resblock_dilation_sizes", ((1, 3, 5),) * 3)),
        leaky_slope=d.get("leaky_relu_slope", 0.1), num_speakers=d.get("num_speakers", 1), speaker_dim=d.get("speaker_embedding_size", 0),
        sampling_rate=d.get("sampling_rate", 16000), noise_scale=d.get("noise_scale", 0.667),
        noise_scale_duration=d.get("noise_scale_duration", 0.8), speaking_rate=d.get("speaking_rate", 1.0))


class _Weights:
    """Named fp32 tensors from a checkpoint (or random ones of the requested shape). Convolutions
    stored with weight normalisation (``parametrizations.weight.original0 / original1`` or
    ``weight_g`` / ``weight_v``) are folded into plain weights on first use."""

    def __init__(self, get, device, seed: int):
        self.get, self.device = get, torch.device(device)
        self.gen = torch.Generator().manual_seed(seed)
        self.cache: dict[str, torch.Tensor] = {}

    def __call__(self, name: str, *shape, init: str = "rand") -> torch.Tensor:
        if name in self.cache:
            return self.cache[name]
        t = self.get(name) if self.get is not None else None
        if t is None and self.get is not None and name.endswith(".weight"):
            stem = name[: -len(".weight")]
            g = self.get(stem + ".parametrizations.weight.original0")
            v = self.get(stem + ".parametrizations.weight.original1")
            if g is None:
                g, v = self.get(stem + ".weight_g"), self.get(stem + ".weight_v")
            if g is not None and v is not None:
                v = v.float()
                t = v * (g.float() / v.flatten(1).norm(dim=1).reshape(-1, *([1] * (v.dim() - 1))))
        if t is None:
            if self.get is not None:
                raise KeyError(name)
            if init == "zeros":
                t = torch.zeros(*shape)
            elif init == "ones":
                t = torch.ones(*shape)
            else:
                fan = 1
                for s in shape[1:]:
                    fan *= s
                t = torch.randn(*shape, generator=self.gen) * (1.0 / max(fan, 1)) ** 0.5
        t = t.float().to(self.device)
        self.cache[name] = t
        return t


# ------------------------------------------------------------------------------------ spline
def _rq_spline_inverse(y: torch.Tensor, uw: torch.Tensor, uh: torch.Tensor, ud: torch.Tensor, tail: float,
                       min_w: float = 1e-3, min_h: float = 1e-3, min_d: float = 1e-3) -> torch.Tensor:
    """Inverse of the monotone rational-quadratic spline on [-tail, tail] (identity outside):
    y [...], unnormalised widths / heights [..., bins] and inner derivatives [..., bins - 1]."""
    inside = (y >= -tail) & (y <= tail)
    out = y.clone()
    if not inside.any():
        return out
    bins = uw.shape[-1]
    const = math.log(math.exp(1 - min_d) - 1)            # boundary derivatives equal 1: the tails join smoothly
    ud = F.pad(ud, (1, 1), value=const)
    yi, uw, uh, ud = y[inside], uw[inside], uh[inside], ud[inside]

    def knots(u, m):
        w = m + (1 - m * bins) * torch.softmax(u, -1)
        c = F.pad(torch.cumsum(w, -1), (1, 0)) * 2 * tail - tail
        c[..., 0], c[..., -1] = -tail, tail
        return c, c[..., 1:] - c[..., :-1]

    cw, w = knots(uw, min_w)
    ch, h = knots(uh, min_h)
    d = min_d + F.softplus(ud)
    loc = ch.clone()
    loc[..., -1] += 1e-6
    idx = ((yi[..., None] >= loc).sum(-1) - 1).clamp(0, bins - 1)[..., None]
    g = lambda t: t.gather(-1, idx)[..., 0]
    in_cw, in_w, in_ch, in_h = g(cw), g(w), g(ch), g(h)
    delta = g(h / w)
    d0, d1 = g(d), g(d[..., 1:])
    s = d0 + d1 - 2 * delta
    t2 = yi - in_ch
    a = in_h * (delta - d0) + t2 * s
    b = in_h * d0 - t2 * s
    c = -delta * t2
    root = (2 * c) / (-b - torch.sqrt((b * b - 4 * a * c).clamp_min(0)))
    out[inside] = root * in_w + in_cw
    return out


# ------------------------------------------------------------------------------------ model
class VitsModel:
    def __init__(self, cfg: VitsConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = _Weights(get, device, seed)
        self.gen = torch.Generator().manual_seed(seed + 1)

    # -- small helpers ----------------------------------------------------------------------
    def _conv(self, x, name, co, ci, k, padding=0, dilation=1, groups=1, bias=True):
        w = self.w(name + ".weight", co, ci // groups, k)
        b = self.w(name + ".bias", co, init="zeros") if bias else None
        return F.conv1d(x, w, b, padding=padding, dilation=dilation, groups=groups)

    def _ln(self, x, name, c):
        """LayerNorm over channels of x [1, C, T]."""
        y = F.layer_norm(x.transpose(1, 2), (c,), self.w(name + ".weight", c, init="ones"), self.w(name + ".bias", c, init="zeros"),
                         self.cfg.eps)
        return y.transpose(1, 2)

    def _randn(self, *shape):
        return torch.randn(*shape, generator=self.gen).to(self.device)

    # -- text encoder -------------------------------------------------------------------------
    def _rel_embeddings(self, name: str, length: int) -> torch.Tensor:
        """The 2 * length - 1 relative embeddings around offset 0 (zero beyond the window)."""
        cfg = self.cfg
        d = cfg.hidden // cfg.heads
        e = self.w(name, 1, 2 * cfg.window + 1, d)[0]
        pad = max(length - (cfg.window + 1), 0)
        if pad:
            e = F.pad(e, (0, 0, pad, pad))
        start = max(cfg.window + 1 - length, 0)
        return e[start:start + 2 * length - 1]

    def _attention(self, x: torch.Tensor, p: str) -> torch.Tensor:
        """x [T, H] -> [T, H]: softmax(q k^T + q . rel_k) (v + rel_v)."""
        cfg = self.cfg
        T, H = x.shape
        h, d = cfg.heads, H // cfg.heads
        lin = lambda n: F.linear(x, self.w(f"{p}{n}.weight", H, H), self.w(f"{p}{n}.bias", H, init="zeros"))
        q = (lin("q_proj") * d ** -0.5).reshape(T, h, d).transpose(0, 1)          # [h, T, d]
        k = lin("k_proj").reshape(T, h, d).transpose(0, 1)
        v = lin("v_proj").reshape(T, h, d).transpose(0, 1)
        idx = torch.arange(T, device=x.device)
        rel = idx[None, :] - idx[:, None] + (T - 1)                                # key - query offset, shifted to >= 0
        logits = q @ k.transpose(1, 2)
        rk = self._rel_embeddings(p + "emb_rel_k", T)                              # [2T - 1, d]
        logits = logits + (q @ rk.t()).gather(2, rel[None].expand(h, T, T))
        probs = torch.softmax(logits, -1)
        out = probs @ v
        rv = self._rel_embeddings(p + "emb_rel_v", T)
        by_offset = torch.zeros(h, T, 2 * T - 1, device=x.device).scatter_add_(2, rel[None].expand(h, T, T), probs)
        out = out + by_offset @ rv
        out = out.transpose(0, 1).reshape(T, H)
        return F.linear(out, self.w(p + "out_proj.weight", H, H), self.w(p + "out_proj.bias", H, init="zeros"))

    def encode_text(self, ids: torch.Tensor):
        """ids [T] -> (hidden [1, H, T], prior mean [1, flow, T], prior log-variance [1, flow, T])."""
        cfg = self.cfg
        H = cfg.hidden
        x = self.w("text_encoder.embed_tokens.weight", cfg.vocab_size, H)[ids.long().to(self.device)] * math.sqrt(H)
        k = cfg.ffn_kernel
        for i in range(cfg.layers):
            p = f"text_encoder.encoder.layers.{i}."
            x = F.layer_norm(x + self._attention(x, p + "attention."), (H,), self.w(p + "layer_norm.weight", H, init="ones"),
                             self.w(p + "layer_norm.bias", H, init="zeros"), cfg.eps)
            y = x.t()[None]
            y = F.pad(y, ((k - 1) // 2, k // 2))
            y = torch.relu(self._conv(y, p + "feed_forward.conv_1", cfg.ffn, H, k))
            y = F.pad(y, ((k - 1) // 2, k // 2))
            y = self._conv(y, p + "feed_forward.conv_2", H, cfg.ffn, k)[0].t()
            x = F.layer_norm(x + y, (H,), self.w(p + "final_layer_norm.weight", H, init="ones"),
                             self.w(p + "final_layer_norm.bias", H, init="zeros"), cfg.eps)
        hid = x.t()[None]
        stats = self._conv(hid, "text_encoder.project", 2 * cfg.flow_size, H, 1)
        return hid, stats[:, : cfg.flow_size], stats[:, cfg.flow_size:]

    # -- duration -----------------------------------------------------------------------------
    def _dds(self, x: torch.Tensor, p: str, c: int, cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Dilated depth-separable convolution stack: depthwise (dilation k^i) -> LN -> GELU ->
        pointwise -> LN -> GELU, residual."""
        cfg = self.cfg
        k = cfg.dds_kernel
        if cond is not None:
            x = x + cond
        for i in range(cfg.dds_layers):
            dil = k ** i
            y = self._conv(x, f"{p}convs_dilated.{i}", c, c, k, padding=(k * dil - dil) // 2, dilation=dil, groups=c)
            y = F.gelu(self._ln(y, f"{p}norms_1.{i}", c))
            y = self._conv(y, f"{p}convs_pointwise.{i}", c, c, 1)
            y = F.gelu(self._ln(y, f"{p}norms_2.{i}", c))
            x = x + y
        return x

    def _conv_flow_reverse(self, z: torch.Tensor, p: str, cond: torch.Tensor) -> torch.Tensor:
        """z [1, 2, T]: the second channel goes back through the spline whose parameters are computed
        from the first channel and the text conditioning."""
        cfg = self.cfg
        c, bins = cfg.hidden, cfg.dp_bins
        first, second = z[:, :1], z[:, 1:]
        h = self._conv(first, p + "conv_pre", c, 1, 1)
        h = self._dds(h, p + "conv_dds.", c, cond)
        h = self._conv(h, p + "conv_proj", 3 * bins - 1, c, 1)
        T = z.shape[-1]
        h = h.reshape(1, 1, 3 * bins - 1, T).permute(0, 1, 3, 2)                   # [1, 1, T, 3 bins - 1]
        scale = math.sqrt(c)
        second = _rq_spline_inverse(second, h[..., :bins] / scale, h[..., bins:2 * bins] / scale, h[..., 2 * bins:],
                                    cfg.dp_tail_bound)
        return torch.cat([first, second], 1)

    def log_durations(self, hidden: torch.Tensor, noise_scale: float) -> torch.Tensor:
        """hidden [1, H, T] -> log duration (frames) per token [1, 1, T]."""
        cfg = self.cfg
        H, T = cfg.hidden, hidden.shape[-1]
        p = "duration_predictor."
        if not cfg.stochastic_duration:
            k, fc = cfg.dp_kernel, cfg.dp_filter
            x = self._ln(torch.relu(self._conv(hidden, p + "conv_1", fc, H, k, padding=k // 2)), p + "norm_1", fc)
            x = self._ln(torch.relu(self._conv(x, p + "conv_2", fc, fc, k, padding=k // 2)), p + "norm_2", fc)
            return self._conv(x, p + "proj", 1, fc, 1)
        x = self._conv(hidden, p + "conv_pre", H, H, 1)
        x = self._dds(x, p + "conv_dds.", H)
        cond = self._conv(x, p + "conv_proj", H, H, 1)
        # flows[0] is the element-wise affine, the rest are spline flows; in reverse the order is
        # last .. first with one spline flow (the second in forward order) left out
        order = list(reversed(range(cfg.dp_flows + 1)))
        order = order[:-2] + [order[-1]]
        z = self._randn(1, 2, T) * noise_scale
        for i in order:
            z = torch.flip(z, [1])
            fp = f"{p}flows.{i}."
            if i == 0:
                z = (z - self.w(fp + "translate", 2, 1, init="zeros")) * torch.exp(-self.w(fp + "log_scale", 2, 1, init="zeros"))
            else:
                z = self._conv_flow_reverse(z, fp, cond)
        return z[:, :1]

    # -- prior flow ---------------------------------------------------------------------------
    def _wavenet(self, x: torch.Tensor, p: str) -> torch.Tensor:
        cfg = self.cfg
        H, k = cfg.hidden, cfg.wavenet_kernel
        out = torch.zeros_like(x)
        for i in range(cfg.wavenet_layers):
            dil = cfg.wavenet_dilation ** i
            a = self._conv(x, f"{p}in_layers.{i}", 2 * H, H, k, padding=(k * dil - dil) // 2, dilation=dil)
            acts = torch.tanh(a[:, :H]) * torch.sigmoid(a[:, H:])
            last = i == cfg.wavenet_layers - 1
            rs = self._conv(acts, f"{p}res_skip_layers.{i}", H if last else 2 * H, H, 1)
            if last:
                out = out + rs
            else:
                x = x + rs[:, :H]
                out = out + rs[:, H:]
        return out

    def flow_reverse(self, z: torch.Tensor) -> torch.Tensor:
        """Prior-space frames [1, flow, L] -> decoder latents: each coupling layer, last first,
        subtracts the mean its WaveNet predicts from the untouched half."""
        cfg = self.cfg
        half = cfg.flow_size // 2
        for i in reversed(range(cfg.prior_flows)):
            z = torch.flip(z, [1])
            p = f"flow.flows.{i}."
            first, second = z[:, :half], z[:, half:]
            h = self._conv(first, p + "conv_pre", cfg.hidden, half, 1)
            mean = self._conv(self._wavenet(h, p + "wavenet."), p + "conv_post", half, cfg.hidden, 1)
            z = torch.cat([first, second - mean], 1)
        return z

    # -- vocoder ------------------------------------------------------------------------------
    def vocode(self, latents: torch.Tensor) -> torch.Tensor:
        """HiFi-GAN: latents [1, flow, L] -> waveform [L * hop]."""
        cfg = self.cfg
        ch = cfg.upsample_initial
        x = self._conv(latents, "decoder.conv_pre", ch, cfg.flow_size, 7, padding=3)
        nk = len(cfg.resblock_kernels)
        for i, (rate, ksz) in enumerate(zip(cfg.upsample_rates, cfg.upsample_kernels)):
            co = ch // 2
            x = F.leaky_relu(x, cfg.leaky_slope)
            x = F.conv_transpose1d(x, self.w(f"decoder.upsampler.{i}.weight", ch, co, ksz),
                                   self.w(f"decoder.upsampler.{i}.bias", co, init="zeros"), stride=rate, padding=(ksz - rate) // 2)
            acc = None
            for j, (rk, dils) in enumerate(zip(cfg.resblock_kernels, cfg.resblock_dilations)):
                p = f"decoder.resblocks.{i * nk + j}."
                y = x
                for m, dil in enumerate(dils):
                    r = self._conv(F.leaky_relu(y, cfg.leaky_slope), f"{p}convs1.{m}", co, co, rk, padding=(rk * dil - dil) // 2, dilation=dil)
                    r = self._conv(F.leaky_relu(r, cfg.leaky_slope), f"{p}convs2.{m}", co, co, rk, padding=(rk - 1) // 2)
                    y = y + r
                acc = y if acc is None else acc + y
            x = acc / nk
            ch = co
        x = self._conv(F.leaky_relu(x), "decoder.conv_post", 1, ch, 7, padding=3, bias=False)
        return torch.tanh(x)[0, 0]

    # -- synthesis ----------------------------------------------------------------------------
    @torch.no_grad()
    def synthesize(self, ids: torch.Tensor, noise_scale: Optional[float] = None, noise_scale_duration: Optional[float] = None,
                   speaking_rate: Optional[float] = None) -> torch.Tensor:
        """Token ids [T] -> waveform [frames * hop] in [-1, 1] at ``cfg.sampling_rate``."""
        cfg = self.cfg
        ns = cfg.noise_scale if noise_scale is None else noise_scale
        nsd = cfg.noise_scale_duration if noise_scale_duration is None else noise_scale_duration
        rate = cfg.speaking_rate if speaking_rate is None else speaking_rate
        hidden, mean, logvar = self.encode_text(ids)
        logd = self.log_durations(hidden, nsd)
        dur = torch.ceil(torch.exp(logd) / rate)[0, 0].clamp_min(0).long()
        if int(dur.sum()) < 1:
            dur[-1] = 1
        token_of_frame = torch.repeat_interleave(torch.arange(dur.numel(), device=self.device), dur)
        mean_f, logvar_f = mean[:, :, token_of_frame], logvar[:, :, token_of_frame]
        z = mean_f + self._randn(*mean_f.shape) * torch.exp(logvar_f) * ns
        return self.vocode(self.flow_reverse(z))
