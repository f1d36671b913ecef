"""JSON grammar constraint for sampling: a byte-level pushdown automaton over JSON text and a
token mask derived from it.

``JsonGrammar.allowed_mask(history_ids)`` returns a boolean mask over the vocabulary of the tokens
that keep the generated text a valid JSON prefix (and allows EOS only once a complete top-level
value has been produced). Same role as the reference's ``JsonGrammarState`` / ``JsonGrammarStep``
(src/HartsyInference.LLM/Sampling/JsonGrammarState.cs), which masks logits before the rest of the
sampler chain runs. Masks are cached per automaton state (mode + the three innermost containers),
so steady-state cost is a dictionary lookup.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

WS = b" \t\n\r"
DIGITS = b"0123456789"

# modes
VALUE, OBJ_FIRST, OBJ_KEY, OBJ_COLON, AFTER_VALUE, ARR_FIRST, STRING, STRING_ESC, STRING_U, NUMBER, LITERAL, DONE = range(12)


class JsonState:
    __slots__ = ("mode", "stack", "is_key", "lit", "lit_pos", "u_left", "num")

    def __init__(self):
        self.mode = VALUE
        self.stack: list[int] = []       # 0 = object, 1 = array
        self.is_key = False
        self.lit = b""
        self.lit_pos = 0
        self.u_left = 0
        self.num = 0                     # number sub-state

    def copy(self) -> "JsonState":
        s = JsonState()
        s.mode, s.stack, s.is_key, s.lit, s.lit_pos, s.u_left, s.num = (self.mode, list(self.stack), self.is_key,
                                                                        self.lit, self.lit_pos, self.u_left, self.num)
        return s

    def key(self):
        return (self.mode, tuple(self.stack[-3:]), len(self.stack) > 3, self.is_key, self.lit, self.lit_pos,
                self.u_left, self.num)

    def complete(self) -> bool:
        return self.mode == DONE or (self.mode == NUMBER and not self.stack and self.num in (1, 2, 4, 7))

    def _end_value(self) -> None:
        self.mode = AFTER_VALUE if self.stack else DONE

    def feed(self, c: int) -> bool:
        """Consume one byte; False = invalid."""
        m = self.mode
        ch = bytes([c])
        if m == STRING:
            if c == 0x22:
                if self.is_key:
                    self.mode, self.is_key = OBJ_COLON, False
                else:
                    self._end_value()
                return True
            if c == 0x5C:
                self.mode = STRING_ESC
                return True
            return c >= 0x20
        if m == STRING_ESC:
            if ch in b'"\\/bfnrt':
                self.mode = STRING
                return True
            if ch == b"u":
                self.mode, self.u_left = STRING_U, 4
                return True
            return False
        if m == STRING_U:
            if ch in b"0123456789abcdefABCDEF":
                self.u_left -= 1
                if self.u_left == 0:
                    self.mode = STRING
                return True
            return False
        if m == NUMBER:
            # num: 0 '-' seen, 1 leading zero, 2 int digits, 3 '.' seen, 4 frac digits, 5 'e' seen, 6 exp sign, 7 exp digits
            n = self.num
            if ch in DIGITS:
                if n == 0:
                    self.num = 1 if ch == b"0" else 2
                elif n == 1:
                    return False
                elif n == 2:
                    pass
                elif n in (3, 4):
                    self.num = 4
                elif n in (5, 6, 7):
                    self.num = 7
                return True
            if ch == b"." and n in (1, 2):
                self.num = 3
                return True
            if ch in b"eE" and n in (1, 2, 4):
                self.num = 5
                return True
            if ch in b"+-" and n == 5:
                self.num = 6
                return True
            if n in (1, 2, 4, 7):        # number ends, re-dispatch the byte
                self._end_value()
                return self.feed(c)
            return False
        if m == LITERAL:
            if self.lit_pos < len(self.lit) and c == self.lit[self.lit_pos]:
                self.lit_pos += 1
                if self.lit_pos == len(self.lit):
                    self._end_value()
                return True
            return False
        if ch in WS:
            return True
        if m in (VALUE, ARR_FIRST):
            if m == ARR_FIRST and ch == b"]":
                self.stack.pop()
                self._end_value()
                return True
            if ch == b"{":
                self.stack.append(0)
                self.mode = OBJ_FIRST
                return True
            if ch == b"[":
                self.stack.append(1)
                self.mode = ARR_FIRST
                return True
            if ch == b'"':
                self.mode, self.is_key = STRING, False
                return True
            if ch == b"-":
                self.mode, self.num = NUMBER, 0
                return True
            if ch in DIGITS:
                self.mode, self.num = NUMBER, (1 if ch == b"0" else 2)
                return True
            for lit in (b"true", b"false", b"null"):
                if c == lit[0]:
                    self.mode, self.lit, self.lit_pos = LITERAL, lit, 1
                    return True
            return False
        if m in (OBJ_FIRST, OBJ_KEY):
            if m == OBJ_FIRST and ch == b"}":
                self.stack.pop()
                self._end_value()
                return True
            if ch == b'"':
                self.mode, self.is_key = STRING, True
                return True
            return False
        if m == OBJ_COLON:
            if ch == b":":
                self.mode = VALUE
                return True
            return False
        if m == AFTER_VALUE:
            top = self.stack[-1]
            if ch == b",":
                self.mode = OBJ_KEY if top == 0 else VALUE
                return True
            if (ch == b"}" and top == 0) or (ch == b"]" and top == 1):
                self.stack.pop()
                self._end_value()
                return True
            return False
        return False                      # DONE: only whitespace (handled above)


class JsonGrammar:
    def __init__(self, tokenizer, eos_ids: Optional[Sequence[int]] = None):
        self.tok = tokenizer
        self.vocab = [tokenizer.token_bytes(i) for i in range(tokenizer.vocab_size)]
        self.eos_ids = list(eos_ids if eos_ids is not None else
                            ([tokenizer.eos_id] if tokenizer.eos_id is not None else []))
        self.special = set(tokenizer.special_ids)
        self._cache: dict = {}

    def state_after(self, ids: Sequence[int]) -> Optional[JsonState]:
        st = JsonState()
        for t in ids:
            if t in self.special:
                continue
            for c in self.vocab[t] if 0 <= t < len(self.vocab) else b"":
                if not st.feed(c):
                    return None
        return st

    def _mask_for(self, st: JsonState) -> torch.Tensor:
        key = st.key()
        m = self._cache.get(key)
        if m is not None:
            return m
        mask = torch.zeros(len(self.vocab), dtype=torch.bool)
        for i, b in enumerate(self.vocab):
            if not b or i in self.special:
                continue
            s = st.copy()
            ok = True
            for c in b:
                if not s.feed(c):
                    ok = False
                    break
            if ok:
                mask[i] = True
        if st.complete():
            for e in self.eos_ids:
                if 0 <= e < len(self.vocab):
                    mask[e] = True
        if len(self._cache) < 4096:
            self._cache[key] = mask
        return mask

    def allowed_mask(self, history_with_prompt: Sequence[int], generated_from: Optional[int] = None) -> torch.Tensor:
        """Mask for the next token. ``history_with_prompt`` may include the prompt; the grammar only
        sees the tokens after ``generated_from`` (default: it tracks the split itself on first use)."""
        if generated_from is None:
            if not hasattr(self, "_prompt_len"):
                self._prompt_len = len(history_with_prompt)
            generated_from = self._prompt_len
        st = self.state_after(history_with_prompt[generated_from:])
        if st is None:                    # should not happen under the mask; fail open on EOS only
            mask = torch.zeros(len(self.vocab), dtype=torch.bool)
            for e in self.eos_ids:
                mask[e] = True
            return mask
        return self._mask_for(st)
