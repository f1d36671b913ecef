"""Layer-split pipeline parallelism for the decoder LLM.

Stage s holds a contiguous range of layers (``DecoderModel(layer_range=...)``), receives the
``(hidden, residual)`` pair of its predecessor over the point-to-point transport (NCCL on GPUs,
gloo on CPU), runs its layers and passes the pair on; the last stage applies the final norm and
the LM head and broadcasts the sampled tokens, so that every stage's scheduler sees the same
sequence state. Only activations of the current step cross the link (2 x T x H bf16).

A step's batch is cut into micro-batches along its sequences (``micro_batches``): stage s works on
micro-batch i while stage s + 1 works on micro-batch i - 1. Transfers are non-blocking (the receive
of micro-batch i + 1 is posted before the layers of micro-batch i run; sends are only waited for at
the end of the step), which on GPUs puts them on the communicator's stream beside the compute
stream. With one micro-batch the stages take turns, as a plain relay would.

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
                 ratios: Optional[Sequence[float]] = None, micro_batches: int = 0):
        self.comm = comm
        # 0 = as many as there are stages (the smallest count that can keep every stage busy)
        self.micro_batches = int(micro_batches) if micro_batches else comm.world
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

    # -- micro-batches
    def split_batch(self, batch: ForwardBatch) -> list[ForwardBatch]:
        """Cut ``batch`` into up to ``micro_batches`` pieces along its sequences (a decode row or a
        prefill sequence is never divided). Batches that carry per-row extras the stages would have to
        re-slice (embeddings, multimodal positions, cross-attention states) stay whole."""
        n_seq = int(batch.kv_lens.shape[0])
        want = min(self.micro_batches, n_seq)
        if want <= 1 or batch.embeds is not None or batch.positions3 is not None or batch.deepstack is not None \
                or batch.cross_states is not None or batch.cross_row_mask is not None:
            return [batch]
        if batch.is_decode:
            bounds = [(n_seq * i) // want for i in range(want + 1)]
            rows = bounds
        else:
            cu = batch.cu_q.tolist()
            total = cu[-1]
            # sequence boundaries closest to equal token shares
            bounds = [0]
            for i in range(1, want):
                target = total * i / want
                j = min(range(bounds[-1] + 1, n_seq), key=lambda k: abs(cu[k] - target), default=None)
                if j is None:
                    break
                bounds.append(j)
            bounds.append(n_seq)
            rows = [cu[b] for b in bounds]
        parts = []
        for i in range(len(bounds) - 1):
            s0, s1, r0, r1 = bounds[i], bounds[i + 1], rows[i], rows[i + 1]
            if s1 <= s0:
                continue
            lr = None
            if batch.logit_rows is not None:
                sel = (batch.logit_rows >= r0) & (batch.logit_rows < r1)
                lr = (batch.logit_rows[sel] - r0).contiguous()
            cu_q = None if batch.cu_q is None else (batch.cu_q[s0:s1 + 1] - batch.cu_q[s0]).contiguous()
            parts.append(ForwardBatch(tokens=batch.tokens[r0:r1].contiguous(), positions=batch.positions[r0:r1].contiguous(),
                                      slot_mapping=batch.slot_mapping[r0:r1].contiguous(),
                                      block_table=batch.block_table[s0:s1].contiguous(), kv_lens=batch.kv_lens[s0:s1].contiguous(),
                                      is_decode=batch.is_decode, cu_q=cu_q,
                                      max_q_len=batch.max_q_len, max_kv_len=batch.max_kv_len, logit_rows=lr))
        return parts or [batch]

    # -- forward
    def forward_hidden(self, batch: ForwardBatch) -> torch.Tensor:
        m = self.model
        h = self.cfg.hidden_size
        parts = self.split_batch(batch)
        sizes = [p.tokens.shape[0] for p in parts]
        recv_bufs = [None] * len(parts)
        recv_work = [None] * len(parts)

        def post_recv(i: int) -> None:
            if not m.first_stage and i < len(parts):
                recv_bufs[i] = torch.empty(2, sizes[i], h, dtype=torch.bfloat16, device=self.device)
                recv_work[i] = self.comm.irecv(recv_bufs[i], self.stage - 1)

        post_recv(0)
        sends, outs = [], []
        for i, mb in enumerate(parts):
            hidden_in = None
            if not m.first_stage:
                recv_work[i].wait()
                hidden_in = (recv_bufs[i][0], recv_bufs[i][1])
            post_recv(i + 1)                      # the next micro-batch arrives while this one is computed
            out = m.forward_hidden(mb, hidden_in=hidden_in)
            if m.last_stage:
                outs.append(out)
            else:
                x, res = out
                if res is None:
                    res = torch.zeros_like(x)
                payload = torch.stack([x, res]).contiguous()
                sends.append((self.comm.isend(payload, self.stage + 1), payload))
        for work, _ in sends:
            work.wait()
        if m.last_stage:
            return outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        # earlier stages have no logits; callers get a placeholder of the right shape
        return torch.zeros(sum(sizes), h, dtype=torch.bfloat16, device=self.device)

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
