"""Prompt weighting: ``(a red fox:1.3)``, ``((emphasis))`` = x1.1 per level, ``[less]`` = /1.1 per level,
``\\(`` for a literal parenthesis. The prompt is parsed into (text, weight) runs; each run's tokens
carry its weight, and the text encoder's token states are scaled around their mean so that the
overall magnitude of the conditioning stays what the encoder produced.

Reference: src/HartsyInference.Diffusion/Prompting/ (prompt weighting / emphasis parser).
"""
from __future__ import annotations

import re
from typing import Callable, Sequence

import torch

_TOKEN = re.compile(r"\\\(|\\\)|\\\[|\\\]|\\\\|\\|\(|\[|:\s*([+-]?(?:\d+\.?\d*|\.\d+))\s*\)|\)|\]|[^\\()\[\]:]+|:")


def parse_prompt_weights(text: str) -> list[tuple[str, float]]:
    """``"a (red:1.5) fox"`` -> ``[("a ", 1.0), ("red", 1.5), (" fox", 1.0)]``."""
    res: list[list] = []
    round_stack: list[int] = []
    square_stack: list[int] = []

    def scale(start: int, m: float) -> None:
        for i in range(start, len(res)):
            res[i][1] *= m

    for m in _TOKEN.finditer(text):
        tok, num = m.group(0), m.group(1)
        if tok.startswith("\\") and len(tok) > 1:
            res.append([tok[1:], 1.0])
        elif tok == "(":
            round_stack.append(len(res))
        elif tok == "[":
            square_stack.append(len(res))
        elif num is not None and round_stack:
            scale(round_stack.pop(), float(num))
        elif tok == ")" and round_stack:
            scale(round_stack.pop(), 1.1)
        elif tok == "]" and square_stack:
            scale(square_stack.pop(), 1 / 1.1)
        else:
            res.append([tok, 1.0])
    for pos in round_stack:          # unclosed brackets still count
        scale(pos, 1.1)
    for pos in square_stack:
        scale(pos, 1 / 1.1)
    merged: list[list] = []
    for t, w in res:
        if not t:
            continue
        if merged and abs(merged[-1][1] - w) < 1e-9:
            merged[-1][0] += t
        else:
            merged.append([t, w])
    return [(t, float(w)) for t, w in merged] or [("", 1.0)]


def token_weights(runs: Sequence[tuple[str, float]], encode: Callable[[str], list[int]], max_len: int) -> tuple[list[int], list[float]]:
    """Tokenise each run by itself (no special tokens) and give its tokens the run's weight."""
    ids: list[int] = []
    ws: list[float] = []
    for text, w in runs:
        piece = encode(text)
        ids += piece
        ws += [w] * len(piece)
    return ids[:max_len], ws[:max_len]


def apply_token_weights(states: torch.Tensor, weights: Sequence[float]) -> torch.Tensor:
    """states [T, D], one weight per leading token (the rest 1.0): scale each token's state, then
    restore the original mean so a heavily weighted prompt does not shift the whole conditioning."""
    w = torch.ones(states.shape[0], dtype=torch.float32, device=states.device)
    n = min(len(weights), states.shape[0])
    w[:n] = torch.tensor(list(weights[:n]), dtype=torch.float32, device=states.device)
    if torch.all(w == 1.0):
        return states
    x = states.float()
    before = x.mean()
    y = x * w[:, None]
    after = y.mean()
    if abs(float(after)) > 1e-12:
        y = y * (before / after)
    return y.to(states.dtype)
