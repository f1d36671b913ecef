"""Fast host path for batch-1 generation: hands a CPU-resident :class:`DecoderModel` of the llama
family to the native decoder (``csrc/runtime/cpu_decoder.cpp``: AVX-512 row kernels, a persistent
thread team, one call per token) instead of running every op through the tensor library.

Eligible models: pre-norm RMSNorm decoders with grouped-query attention, full split-half rotary
embedding, SwiGLU feed-forward, bf16 / fp32 weights held as plain matrices (no fp8, no MoE, no
sliding window / soft-cap / sandwich norms). Everything else keeps the general path. fp32 math on
fp32 copies of the weights, like the reference's CPU backend
(src/HartsyInference.Cpu/Kernels/MatMulKernels.cs:106, Threading/ComputeThreadPool.cs).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from ... import runtime
from .transformer import DecoderModel


def eligible(model: DecoderModel) -> bool:
    cfg = model.cfg
    if model.device.type != "cpu" or model.tp != 1 or not (model.first_stage and model.last_stage):
        return False
    if cfg.general_path or cfg.mla is not None or (cfg.moe is not None and cfg.moe.num_experts > 0):
        return False
    if not cfg.gated_ffn or cfg.activation != "silu" or cfg.post_norms or cfg.norm_plus_one or cfg.qk_norm:
        return False
    if cfg.rotary_dim != cfg.head_dim or cfg.rope_style != 0 or cfg.rope_scaling.kind != "none" or not cfg.use_rope:
        return False
    if cfg.attn_softcap or cfg.logit_softcap or cfg.embed_scale != 1.0 or cfg.residual_multiplier != 1.0 or cfg.attn_scale > 0:
        return False
    if cfg.embedding_multiplier != 1.0 or cfg.logits_scale != 1.0 or cfg.attn_sinks or cfg.alibi or cfg.learned_positions:
        return False
    if any(cfg.layer_window(i) > 0 for i in range(cfg.num_layers)):
        return False
    return all(lw.qkv is not None and lw.o is not None and lw.gate_up is not None and lw.down is not None
               and not lw.qkv.is_fp8 and lw.o.bias is None and lw.down.bias is None and lw.gate_up.bias is None
               for lw in model.layers)


class CpuDecoder:
    def __init__(self, model: DecoderModel, max_positions: int = 4096, threads: int = 0):
        if not eligible(model):
            raise ValueError("this model does not fit the native host decoder (see cpu_decoder.eligible)")
        L = runtime.lib()
        vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
        L.b200_cpu_decoder_create.restype = vp
        L.b200_cpu_decoder_create.argtypes = [i32] * 8 + [f32, f32, i32]
        L.b200_cpu_decoder_free.argtypes = [vp]
        L.b200_cpu_decoder_set_globals.argtypes = [vp, vp, vp, vp]
        L.b200_cpu_decoder_set_layer.restype = i32
        L.b200_cpu_decoder_set_layer.argtypes = [vp, i32] + [vp] * 7
        L.b200_cpu_decoder_forward.restype = i32
        L.b200_cpu_decoder_forward.argtypes = [vp, i32, i32, vp]
        L.b200_cpu_decoder_threads.restype = i32
        L.b200_cpu_decoder_threads.argtypes = [vp]
        L.b200_cpu_decoder_simd.restype = i32
        self._L = L
        cfg = model.cfg
        self.cfg = cfg
        self.max_positions = max_positions
        self._h = L.b200_cpu_decoder_create(cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim,
                                            cfg.ffn_size, cfg.vocab_size, max_positions, cfg.rms_eps, cfg.rope_theta, threads)
        if not self._h:
            raise ValueError("bad decoder shape")
        # fp32 copies kept alive here; the native side only borrows the pointers
        self._keep: list[torch.Tensor] = []

        def f32t(t: Optional[torch.Tensor]) -> Optional[int]:
            if t is None:
                return None
            c = t.detach().to(torch.float32).contiguous()
            self._keep.append(c)
            return c.data_ptr()

        emb = f32t(model.embed)
        head = emb if model.lm_head.weight.data_ptr() == model.embed.data_ptr() else f32t(model.lm_head.weight[: cfg.vocab_size])
        L.b200_cpu_decoder_set_globals(self._h, emb, head, f32t(model.final_norm))
        for i, lw in enumerate(model.layers):
            rc = L.b200_cpu_decoder_set_layer(self._h, i, f32t(lw.in_norm), f32t(lw.qkv.weight), f32t(lw.qkv.bias),
                                              f32t(lw.o.weight), f32t(lw.post_norm), f32t(lw.gate_up.weight),
                                              f32t(lw.down.weight))
            assert rc == 0
        self.threads = L.b200_cpu_decoder_threads(self._h)
        self.simd_bits = L.b200_cpu_decoder_simd()
        self.pos = 0

    def reset(self) -> None:
        self.pos = 0

    def step(self, token: int, want_logits: bool = False):
        """Feed one token at the next position; returns the greedy next token (and the logits)."""
        if self.pos >= self.max_positions:
            raise ValueError("context full")
        out = torch.empty(self.cfg.vocab_size, dtype=torch.float32) if want_logits else None
        nxt = self._L.b200_cpu_decoder_forward(self._h, int(token), self.pos, out.data_ptr() if out is not None else None)
        if nxt < 0:
            raise ValueError("bad token or position")
        self.pos += 1
        return (nxt, out) if want_logits else nxt

    def generate(self, prompt: Sequence[int], max_new_tokens: int) -> list[int]:
        """Greedy continuation of ``prompt`` (the prompt is fed token by token)."""
        self.reset()
        nxt = 0
        for t in prompt:
            nxt = self.step(t)
        out = []
        for _ in range(max_new_tokens):
            out.append(nxt)
            if len(out) == max_new_tokens:
                break
            nxt = self.step(nxt)
        return out

    def close(self) -> None:
        if self._h:
            self._L.b200_cpu_decoder_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
