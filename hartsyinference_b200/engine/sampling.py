"""Token sampling.

Order of the chain follows the reference's ``SamplerChain``
(src/HartsyInference.LLM/Sampling/SamplerChain.cs:26-85): grammar mask -> repetition penalty ->
temperature -> top-k -> top-p -> min-p -> seeded multinomial; greedy requests still receive the
logit-adjusting steps and then take the argmax. Everything runs on the device that holds the
logits; only the chosen ids are read back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch

from .. import ops


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.95
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 4096
    seed: Optional[int] = None
    greedy: bool = False
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    # optional callable(list_of_generated_ids) -> bool mask tensor [vocab] of allowed tokens
    logits_mask: Optional[Callable[[Sequence[int]], torch.Tensor]] = None

    @property
    def is_greedy(self) -> bool:
        return self.greedy or self.temperature <= 0.0

    @property
    def needs_logits(self) -> bool:
        return (not self.is_greedy) or self.repetition_penalty != 1.0 or self.logits_mask is not None


def sample_row(logits: torch.Tensor, p: SamplingParams, history: Sequence[int],
               generator: Optional[torch.Generator]) -> int:
    """Sample one token from fp32 logits [vocab] for one request."""
    lg = logits.float().clone()
    if p.logits_mask is not None:
        mask = p.logits_mask(history).to(lg.device)
        lg = lg.masked_fill(~mask, float("-inf"))
    if p.repetition_penalty != 1.0 and len(history) > 0:
        h = torch.tensor(list(history)[-4096:], dtype=torch.int32, device=lg.device)[None]
        ops.repetition_penalty_(lg[None], h, torch.tensor([h.shape[1]], dtype=torch.int32, device=lg.device),
                                torch.tensor([p.repetition_penalty], dtype=torch.float32, device=lg.device))
    if p.is_greedy:
        return int(ops.argmax(lg[None])[0])
    lg = lg / max(p.temperature, 1e-6)
    if p.top_k and p.top_k > 0 and p.top_k < lg.numel():
        kth = torch.topk(lg, p.top_k).values[-1]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    probs = torch.softmax(lg, dim=-1)
    if 0.0 < p.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cum = torch.cumsum(sp, dim=-1)
        drop = cum - sp > p.top_p
        sp = sp.masked_fill(drop, 0.0)
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
    if p.min_p > 0.0:
        probs = probs.masked_fill(probs < p.min_p * probs.max(), 0.0)
    probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=generator)[0])
