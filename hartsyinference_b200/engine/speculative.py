"""Prompt-lookup speculative decoding for a single greedy request.

The draft comes from the request's own context: the last ``ngram`` tokens are searched (most
recent match first, within ``lookback`` tokens) and the tokens that followed the match are
proposed. One forward pass over ``[last token, draft...]`` (causal, on top of the cached prefix)
verifies the whole draft: position i's greedy token must equal draft token i. The accepted prefix
plus the first correction are kept; the KV entries of rejected positions are cut off with the
allocator's ``truncate``. Outputs are identical to plain greedy decoding of the same model.

Reference behaviour: src/HartsyInference.LLM/Generation/TextGenerationPipeline.cs
(GenerateSpeculative:403-463; n-gram 3, draft length 8, look-back 4096).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch

from ..models.llm.transformer import ForwardBatch
from .sampling import SamplingParams


@dataclass
class SpeculativeStats:
    forward_passes: int = 0
    drafted: int = 0
    accepted: int = 0

    @property
    def tokens_per_pass(self) -> float:
        return 0.0 if self.forward_passes == 0 else (self.accepted + self.forward_passes) / self.forward_passes


def find_draft(tokens: Sequence[int], ngram: int = 3, max_draft: int = 8, lookback: int = 4096) -> list[int]:
    """Tokens that followed the most recent earlier occurrence of the last ``ngram`` tokens."""
    n = len(tokens)
    if n <= ngram:
        return []
    key = list(tokens[n - ngram:])
    lo = max(0, n - lookback)
    for start in range(n - ngram - 1, lo - 1, -1):
        if list(tokens[start:start + ngram]) == key:
            follow = list(tokens[start + ngram:start + ngram + max_draft])
            if follow:
                return follow
    return []


def _forward_chunk(engine, seq: int, toks: Sequence[int], start: int) -> torch.Tensor:
    """Appends ``toks`` at positions [start, start + len) of sequence ``seq`` and returns the hidden
    states of all their rows."""
    count = len(toks)
    page = engine.page
    if engine.kv.append(seq, count) < 0:
        raise RuntimeError("KV pool exhausted")
    engine.h_tokens[:count] = torch.tensor(list(toks), dtype=torch.int32)
    engine.h_positions[:count] = torch.arange(start, start + count, dtype=torch.int32)
    engine._fill_table(0, seq)
    pos = torch.arange(start, start + count, dtype=torch.int64)
    engine.h_slots[:count] = engine.h_table[0][(pos // page)].to(torch.int64) * page + pos % page
    engine.h_cu_q[0] = 0
    engine.h_cu_q[1] = count
    engine.h_kv_lens[0] = start + count
    batch = ForwardBatch(tokens=engine._to_device(engine.h_tokens, count),
                         positions=engine._to_device(engine.h_positions, count),
                         slot_mapping=engine._to_device(engine.h_slots, count),
                         block_table=engine._to_device(engine.h_table, 1),
                         kv_lens=engine._to_device(engine.h_kv_lens, 1), is_decode=False,
                         cu_q=engine._to_device(engine.h_cu_q, 2), max_q_len=count, max_kv_len=start + count)
    return engine.model.forward_hidden(batch)


def generate_speculative(engine, prompt: Sequence[int], params: Optional[SamplingParams] = None, *,
                         ngram: int = 3, max_draft: int = 8, lookback: int = 4096,
                         on_token: Optional[Callable[[int], None]] = None) -> tuple[list[int], SpeculativeStats]:
    """Greedy generation with prompt-lookup drafts. Returns (generated ids, statistics)."""
    params = params or SamplingParams(greedy=True)
    if params.needs_logits:
        raise ValueError("speculative decoding verifies greedy tokens; use a greedy request")
    prompt = list(prompt)
    limit = min(params.max_tokens, engine.max_model_len - len(prompt))
    if limit <= 0:
        raise ValueError("prompt leaves no room for generation")
    max_draft = min(max_draft, max(0, engine.prefill_chunk - 1))
    seq = (1 << 30) + engine._next_id
    engine._next_id += 1
    stats = SpeculativeStats()
    eos = set(engine.model.cfg.eos_token_ids) | set(params.stop_token_ids)
    out: list[int] = []
    try:
        # prompt in chunks of the engine's prefill budget
        hidden = None
        for c0 in range(0, len(prompt), engine.prefill_chunk):
            hidden = _forward_chunk(engine, seq, prompt[c0:c0 + engine.prefill_chunk], c0)
        stats.forward_passes += 1
        nxt = int(engine.model.greedy_tokens(hidden[-1:].contiguous())[0])
        cached = len(prompt)

        def emit(tok: int) -> bool:
            out.append(tok)
            if on_token is not None:
                on_token(tok)
            return (not params.ignore_eos and tok in eos) or len(out) >= limit

        done = emit(nxt)
        while not done:
            ctx = prompt + out
            draft = find_draft(ctx, ngram, max_draft, lookback)
            draft = draft[:max(0, limit - len(out) - 1)]
            # rows: [last emitted token, draft...]; row i predicts the token after position cached + i
            hidden = _forward_chunk(engine, seq, [out[-1]] + draft, cached)
            stats.forward_passes += 1
            stats.drafted += len(draft)
            pred = engine.model.greedy_tokens(hidden.contiguous()).tolist()
            n_ok = 0
            while n_ok < len(draft) and pred[n_ok] == draft[n_ok]:
                n_ok += 1
            stats.accepted += n_ok
            # keep the verified positions: the last emitted token + n_ok accepted draft tokens
            cached += 1 + n_ok
            engine.kv.truncate(seq, cached)
            for tok in draft[:n_ok] + [pred[n_ok]]:
                done = emit(int(tok))
                if done:
                    break
    finally:
        engine.kv.free(seq)
    return out, stats
