"""Layer-split pipeline parallelism for the decoder LLM.

Stage s holds a contiguous range of layers (``DecoderModel(layer_range=...)``), receives the
``(hidden, residual)`` pair of its predecessor over the point-to-point transport (NCCL on GPUs,
gloo on CPU), runs its layers and passes the pair on; the last stage applies the final norm and
the LM head and broadcasts the sampled tokens, so that every stage's scheduler sees the same
sequence state. Only activations of the current step cross the link (2 x T x H bf16).

``PipelinedModel`` has the surface the serving engine uses (``forward_hidden``, ``greedy_tokens``,
``full_logits``, ``alloc_kv`` ...), so an engine per stage runs unchanged.

Reference: src/HartsyInference.LLM/Transformer/GenericTransformer.cs (ForwardEmbedsStaged:309-361),
LlmPlacement.cs (contiguous layer ranges per device, weighted by ShardRatios).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..models.llm.config import TransformerConfig
from ..models.llm.transformer import DecoderModel, ForwardBatch
from .comm import Comm


def split_layers(num_layers: int, stages: int, ratios: Optional[Sequence[float]] = None) -> list[tuple[int, int]]:
    """Contiguous layer ranges, proportional to ``ratios`` (largest-remainder rounding, every
    stage gets at least one layer)."""
    if stages < 1 or stages > num_layers:
        raise ValueError(f"cannot split {num_layers} layers over {stages} stages")
    ratios = list(ratios) if ratios else [1.0] * stages
    if len(ratios) != stages or any(r <= 0 for r in ratios):
        raise ValueError("one positive ratio per stage")
    total = sum(ratios)
    ideal = [num_layers * r / total for r in ratios]
    counts = [max(1, int(x)) for x in ideal]
    while sum(counts) > num_layers:
        i = max(range(stages), key=lambda j: counts[j] - ideal[j] if counts[j] > 1 else -1e9)
        counts[i] -= 1
    order = sorted(range(stages), key=lambda j: ideal[j] - counts[j], reverse=True)
    k = 0
    while sum(counts) < num_layers:
        counts[order[k % stages]] += 1
        k += 1
    out, a = [], 0
    for c in counts:
        out.append((a, a + c))
        a += c
    return out


class PipelinedModel:
    """One pipeline stage with the model surface of :class:`DecoderModel`."""

    def __init__(self, cfg: TransformerConfig, comm: Comm, device="cpu", fp8: bool = False,
                 ratios: Optional[Sequence[float]] = None):
        self.comm = comm
        self.stage, self.stages = comm.rank, comm.world
        self.ranges = split_layers(cfg.num_layers, self.stages, ratios)
        self.model = DecoderModel(cfg, device, fp8=fp8, layer_range=self.ranges[self.stage])
        self.cfg = cfg
        self.device = self.model.device
        self.fp8 = fp8

    # -- weights / cache: straight through to the stage's model
    def random_init(self, seed: int = 0, std: float = 0.02) -> None:
        self.model.random_init(seed, std)

    def load_state_dict(self, get) -> None:
        self.model.load_state_dict(get)

    def weight_bytes(self) -> int:
        return self.model.weight_bytes()

    def kv_bytes_per_page(self, page: int) -> int:
        return self.model.kv_bytes_per_page(page)

    def alloc_kv(self, num_pages: int, page: int = 16):
        return self.model.alloc_kv(num_pages, page)

    @property
    def kv_cache(self):
        return self.model.kv_cache

    # -- forward
    def forward_hidden(self, batch: ForwardBatch) -> torch.Tensor:
        m = self.model
        hidden_in = None
        t = batch.tokens.shape[0] if batch.tokens is not None else batch.embeds.shape[0]
        h = self.cfg.hidden_size
        if not m.first_stage:
            buf = torch.empty(2, t, h, dtype=torch.bfloat16, device=self.device)
            self.comm.recv(buf, self.stage - 1)
            hidden_in = (buf[0], buf[1])
        out = m.forward_hidden(batch, hidden_in=hidden_in)
        if m.last_stage:
            return out
        x, res = out
        if res is None:
            res = torch.zeros_like(x)
        self.comm.send(torch.stack([x, res]).contiguous(), self.stage + 1)
        # earlier stages have no logits; callers get a placeholder of the right shape
        return torch.zeros(t, h, dtype=torch.bfloat16, device=self.device)

    def greedy_tokens(self, hidden: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = hidden.shape[0]
        tok = self.model.greedy_tokens(hidden) if self.model.last_stage else \
            torch.zeros(n, dtype=torch.int32, device=self.device)
        tok = tok.to(torch.int32).contiguous()
        self.comm.broadcast(tok, src=self.stages - 1)
        if out is not None:
            out.copy_(tok)
            return out
        return tok

    def full_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        n = hidden.shape[0]
        if self.model.last_stage:
            lg = self.model.full_logits(hidden).float().contiguous()
        else:
            lg = torch.zeros(n, self.cfg.vocab_size, dtype=torch.float32, device=self.device)
        self.comm.broadcast(lg, src=self.stages - 1)
        return lg
