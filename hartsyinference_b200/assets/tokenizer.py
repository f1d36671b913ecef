"""Tokenizers: byte-level BPE (``tokenizer.json`` of Llama-3 / Qwen / GPT-2 style models) and
SentencePiece-style score BPE (vocabularies embedded in GGUF files), with special-token splitting
and an incremental, UTF-8-safe detokenizer for streaming.

The merge loops run in C++ (``csrc/runtime/tokenizer.cpp``); this module does pre-tokenisation
(regex), special tokens, and decoding. Reference: src/HartsyInference.ModelAssets/Tokenizers/
(BPE for Llama / Qwen2/3 / GPT-OSS, SentencePiece for Gemma / T5, ``Gguf/SpmGguf``,
``HfTokenizerJson``).
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path
from typing import Iterable, Optional, Sequence

import numpy as np

try:
    import regex as _re
except ImportError:  # pragma: no cover
    import re as _re

from .. import runtime

GPT2_PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
LLAMA3_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                  r"\s*[\r\n]+|\s+(?!\S)|\s+")
QWEN2_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                 r"\s*[\r\n]+|\s+(?!\S)|\s+")


def _bytes_to_unicode() -> dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, (chr(c) for c in cs)))


_B2U = _bytes_to_unicode()
_U2B = {v: k for k, v in _B2U.items()}
_bound = False


def _lib():
    global _bound
    L = runtime.lib()
    if not _bound:
        vp, i32 = C.c_void_p, C.c_int32
        for name, res, args in (
            ("b200_tok_create", vp, [vp, vp, i32, vp, i32]), ("b200_tok_destroy", None, [vp]),
            ("b200_tok_add_merge", None, [vp, i32, i32, i32]), ("b200_tok_set_byte_token", None, [vp, i32, i32]),
            ("b200_tok_lookup", i32, [vp, C.c_char_p, i32]),
            ("b200_tok_encode_rank", i32, [vp, C.c_char_p, i32, vp, i32]),
            ("b200_tok_encode_score", i32, [vp, C.c_char_p, i32, vp, i32]),
            ("b200_tok_bytes", i32, [vp, i32, vp, i32]), ("b200_tok_size", i32, [vp]),
        ):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return L


class Tokenizer:
    """``kind`` is ``"bpe"`` (byte-level rank BPE) or ``"spm"`` (score BPE)."""

    def __init__(self, kind: str, token_bytes: Sequence[bytes], *, merges: Optional[Sequence[tuple[int, int]]] = None,
                 scores: Optional[Sequence[float]] = None, special_tokens: Optional[dict[str, int]] = None,
                 pattern: str = GPT2_PATTERN, bos_id: Optional[int] = None, eos_id: Optional[int] = None,
                 add_bos: bool = False, add_space_prefix: bool = True, unk_id: int = -1,
                 byte_fallback: Optional[dict[int, int]] = None):
        self.kind = kind
        self.vocab_bytes = list(token_bytes)
        self.special_tokens = dict(special_tokens or {})
        self.special_ids = set(self.special_tokens.values())
        self.bos_id, self.eos_id, self.add_bos = bos_id, eos_id, add_bos
        self.add_space_prefix = add_space_prefix
        self._pattern = _re.compile(pattern)
        L = _lib()
        self._L = L
        blob = b"".join(self.vocab_bytes)
        lens = np.asarray([len(b) for b in self.vocab_bytes], dtype=np.int32)
        sc = np.asarray(scores, dtype=np.float32) if scores is not None else None
        self._h = L.b200_tok_create(blob, lens.ctypes.data, len(self.vocab_bytes),
                                    sc.ctypes.data if sc is not None else None, unk_id)
        if kind == "bpe":
            for b in range(256):
                tid = L.b200_tok_lookup(self._h, bytes([b]), 1)
                if tid >= 0:
                    L.b200_tok_set_byte_token(self._h, b, tid)
            for rank, (a, b) in enumerate(merges or ()):
                L.b200_tok_add_merge(self._h, a, b, rank)
        else:
            for b, tid in (byte_fallback or {}).items():
                L.b200_tok_set_byte_token(self._h, b, tid)
        if self.special_tokens:
            alt = "|".join(_re.escape(s) for s in sorted(self.special_tokens, key=len, reverse=True))
            self._special_re = _re.compile(f"({alt})")
        else:
            self._special_re = None
        self._buf = (C.c_int32 * 4096)()

    def __del__(self):  # pragma: no cover
        try:
            if self._h:
                self._L.b200_tok_destroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def vocab_size(self) -> int:
        return len(self.vocab_bytes)

    # ------------------------------------------------------------------------------ encode
    def _encode_piece(self, data: bytes, fn) -> list[int]:
        cap = max(len(data), 1)
        buf = self._buf if cap <= 4096 else (C.c_int32 * cap)()
        n = fn(self._h, data, len(data), buf, cap)
        if n < 0:
            raise ValueError("tokenizer buffer overflow")
        return list(buf[:n])

    def _encode_ordinary(self, text: str) -> list[int]:
        out: list[int] = []
        if not text:
            return out
        if self.kind == "bpe":
            for m in self._pattern.finditer(text):
                out.extend(self._encode_piece(m.group().encode("utf-8"), self._L.b200_tok_encode_rank))
        else:
            t = text.replace(" ", "▁")
            out.extend(self._encode_piece(t.encode("utf-8"), self._L.b200_tok_encode_score))
        return out

    def encode(self, text: str, add_special: bool = True, allow_special: bool = True) -> list[int]:
        ids: list[int] = []
        if add_special and self.add_bos and self.bos_id is not None:
            ids.append(self.bos_id)
        first = True
        parts = self._special_re.split(text) if (self._special_re is not None and allow_special) else [text]
        for part in parts:
            if not part:
                continue
            if allow_special and part in self.special_tokens:
                ids.append(self.special_tokens[part])
            else:
                if self.kind == "spm" and self.add_space_prefix and first:
                    part = " " + part
                ids.extend(self._encode_ordinary(part))
            first = False
        return ids

    # ------------------------------------------------------------------------------ decode
    def token_bytes(self, tid: int) -> bytes:
        if 0 <= tid < len(self.vocab_bytes):
            return self.vocab_bytes[tid]
        return b""

    def decode_bytes(self, ids: Iterable[int], skip_special: bool = True) -> bytes:
        out = bytearray()
        for t in ids:
            if skip_special and t in self.special_ids:
                continue
            out += self.token_bytes(t)
        return bytes(out)

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        text = self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")
        if self.kind == "spm":
            text = text.replace("▁", " ")
            if self.add_space_prefix and text.startswith(" "):
                text = text[1:]
        return text

    def stream_decoder(self) -> "StreamDecoder":
        return StreamDecoder(self)

    # ------------------------------------------------------------------------------ loaders
    @staticmethod
    def from_hf_json(path: str | Path) -> "Tokenizer":
        """Load a Hugging Face ``tokenizer.json`` with a BPE model (byte-level or byte-fallback)."""
        d = json.loads(Path(path).read_text(encoding="utf-8"))
        model = d["model"]
        if model.get("type") != "BPE":
            raise ValueError(f"unsupported tokenizer model {model.get('type')}")
        vocab: dict[str, int] = model["vocab"]
        added = {t["content"]: t["id"] for t in d.get("added_tokens", [])}
        size = max(list(vocab.values()) + list(added.values())) + 1
        pre = json.dumps(d.get("pre_tokenizer") or {})
        byte_level = "ByteLevel" in pre or "ByteLevel" in json.dumps(d.get("decoder") or {})
        toks: list[bytes] = [b""] * size
        for s, i in vocab.items():
            toks[i] = bytes(_U2B[c] for c in s) if byte_level and all(c in _U2B for c in s) else s.encode("utf-8")
        for s, i in added.items():
            toks[i] = s.encode("utf-8")
        merges = []
        for m in model.get("merges", []):
            a, b = m.split(" ", 1) if isinstance(m, str) else m
            if a in vocab and b in vocab:
                merges.append((vocab[a], vocab[b]))
        pattern = GPT2_PATTERN
        mobj = _re.search(r'"Regex":\s*"((?:[^"\\]|\\.)*)"', pre)
        if mobj:
            try:
                cand = json.loads('"' + mobj.group(1) + '"')
                _re.compile(cand)
                pattern = cand
            except Exception:
                pass
        if byte_level:
            return Tokenizer("bpe", toks, merges=merges, special_tokens=added, pattern=pattern)
        # SentencePiece-BPE exported to tokenizer.json (Llama-2 / Mistral): score = -rank
        scores = [0.0] * size
        for rank, (a, b) in enumerate(merges):
            mid = vocab.get(next(k for k, v in vocab.items() if v == a) + next(k for k, v in vocab.items() if v == b))
            if mid is not None:
                scores[mid] = -float(rank)
        fb = {b: vocab[f"<0x{b:02X}>"] for b in range(256) if f"<0x{b:02X}>" in vocab}
        return Tokenizer("spm", toks, scores=scores, special_tokens=added, byte_fallback=fb,
                         unk_id=vocab.get("<unk>", -1))

    @staticmethod
    def from_gguf_metadata(md: dict) -> "Tokenizer":
        """Build from ``tokenizer.ggml.*`` keys (model ``gpt2`` = byte-level BPE, ``llama`` = score BPE)."""
        tokens: list[str] = md["tokenizer.ggml.tokens"]
        kind = md.get("tokenizer.ggml.model", "llama")
        types = md.get("tokenizer.ggml.token_type") or [1] * len(tokens)
        bos, eos = md.get("tokenizer.ggml.bos_token_id"), md.get("tokenizer.ggml.eos_token_id")
        add_bos = bool(md.get("tokenizer.ggml.add_bos_token", kind == "llama"))
        special = {t: i for i, (t, ty) in enumerate(zip(tokens, types)) if ty in (3, 4) and t}
        if kind == "gpt2":
            toks = [bytes(_U2B[c] for c in t) if all(c in _U2B for c in t) else t.encode("utf-8") for t in tokens]
            index = {t: i for i, t in enumerate(tokens)}
            merges = []
            for m in md.get("tokenizer.ggml.merges", []):
                a, b = m.split(" ", 1)
                if a in index and b in index:
                    merges.append((index[a], index[b]))
            pre = md.get("tokenizer.ggml.pre", "")
            pattern = LLAMA3_PATTERN if "llama" in pre else QWEN2_PATTERN if "qwen" in pre else GPT2_PATTERN
            return Tokenizer("bpe", toks, merges=merges, special_tokens=special, pattern=pattern, bos_id=bos,
                             eos_id=eos, add_bos=add_bos)
        toks, fb = [], {}
        for i, (t, ty) in enumerate(zip(tokens, types)):
            if ty == 6 and len(t) == 6 and t.startswith("<0x"):
                b = int(t[3:5], 16)
                fb[b] = i
                toks.append(bytes([b]))
            else:
                toks.append(t.encode("utf-8"))
        scores = md.get("tokenizer.ggml.scores") or [0.0] * len(tokens)
        return Tokenizer("spm", toks, scores=scores, special_tokens=special, bos_id=bos, eos_id=eos, add_bos=add_bos,
                         add_space_prefix=bool(md.get("tokenizer.ggml.add_space_prefix", True)),
                         unk_id=md.get("tokenizer.ggml.unknown_token_id", -1) or -1, byte_fallback=fb)


class StreamDecoder:
    """Feed token ids one at a time; get back only complete UTF-8 text (no broken code points)."""

    def __init__(self, tok: Tokenizer):
        self.tok = tok
        self._pending = b""
        self._first = True

    def push(self, tid: int) -> str:
        if tid in self.tok.special_ids:
            return ""
        self._pending += self.tok.token_bytes(tid)
        # emit the longest prefix that is valid UTF-8
        end = len(self._pending)
        for cut in range(0, min(4, end) + 1):
            try:
                text = self._pending[:end - cut].decode("utf-8")
                self._pending = self._pending[end - cut:]
                break
            except UnicodeDecodeError:
                continue
        else:
            text = self._pending.decode("utf-8", errors="replace")
            self._pending = b""
        if self.tok.kind == "spm":
            text = text.replace("▁", " ")
            if self._first and self.tok.add_space_prefix and text.startswith(" "):
                text = text[1:]
        if text:
            self._first = False
        return text

    def flush(self) -> str:
        text = self._pending.decode("utf-8", errors="replace")
        self._pending = b""
        return text


class ByteTokenizer(Tokenizer):
    """Trivial tokenizer (one token per byte + optional specials) for synthetic checkpoints and tests
    (the role of the reference's ``StubTokenizer``)."""

    def __init__(self, specials: Optional[dict[str, int]] = None, vocab_size: int = 256):
        toks = [bytes([i]) for i in range(256)] + [b""] * max(0, vocab_size - 256)
        for s, i in (specials or {}).items():
            if i >= len(toks):
                toks += [b""] * (i + 1 - len(toks))
            toks[i] = s.encode()
        super().__init__("bpe", toks, merges=[], special_tokens=specials or {}, pattern=r"(?s).")


class WordPieceTokenizer:
    """BERT WordPiece: lower-casing / accent stripping (optional), whitespace + punctuation
    pre-tokenisation, greedy longest-match-first pieces with the ``##`` continuation prefix,
    ``[CLS] ... [SEP]`` framing. Loads ``vocab.txt`` or a ``tokenizer.json`` whose model type is
    WordPiece (reference: the BERT tokenizer under src/HartsyInference.ModelAssets/Tokenizers/)."""

    def __init__(self, vocab: list[str], lower: bool = True, unk: str = "[UNK]", cls: str = "[CLS]", sep: str = "[SEP]",
                 max_word_chars: int = 100):
        self.vocab = vocab
        self.index = {t: i for i, t in enumerate(vocab)}
        self.lower = lower
        self.unk_id = self.index.get(unk, 0)
        self.cls_id = self.index.get(cls)
        self.sep_id = self.index.get(sep)
        self.max_word_chars = max_word_chars

    @staticmethod
    def from_dir(path) -> "WordPieceTokenizer":
        import json
        from pathlib import Path
        p = Path(path)
        lower = True
        cfg = p / "tokenizer_config.json"
        if cfg.exists():
            lower = bool(json.loads(cfg.read_text()).get("do_lower_case", True))
        if (p / "vocab.txt").exists():
            vocab = (p / "vocab.txt").read_text(encoding="utf-8").split("\n")
            if vocab and vocab[-1] == "":
                vocab.pop()
            return WordPieceTokenizer(vocab, lower)
        tj = json.loads((p / "tokenizer.json").read_text(encoding="utf-8"))
        if tj.get("model", {}).get("type") != "WordPiece":
            raise ValueError("tokenizer.json does not hold a WordPiece model")
        items = sorted(tj["model"]["vocab"].items(), key=lambda kv: kv[1])
        norm = tj.get("normalizer") or {}
        return WordPieceTokenizer([k for k, _ in items], bool(norm.get("lowercase", True)))

    @staticmethod
    def _is_punct(ch: str) -> bool:
        import unicodedata
        cp = ord(ch)
        if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
            return True
        return unicodedata.category(ch).startswith("P")

    def _basic(self, text: str) -> list[str]:
        import unicodedata
        if self.lower:
            text = unicodedata.normalize("NFD", text.lower())
            text = "".join(c for c in text if unicodedata.category(c) != "Mn")
        words, cur = [], []
        for ch in text:
            if ch.isspace():
                if cur:
                    words.append("".join(cur)); cur = []
            elif self._is_punct(ch) or 0x4E00 <= ord(ch) <= 0x9FFF:
                if cur:
                    words.append("".join(cur)); cur = []
                words.append(ch)
            else:
                cur.append(ch)
        if cur:
            words.append("".join(cur))
        return words

    def _pieces(self, word: str) -> list[int]:
        if len(word) > self.max_word_chars:
            return [self.unk_id]
        out, start = [], 0
        while start < len(word):
            end, cur = len(word), None
            while start < end:
                sub = word[start:end] if start == 0 else "##" + word[start:end]
                if sub in self.index:
                    cur = self.index[sub]
                    break
                end -= 1
            if cur is None:
                return [self.unk_id]
            out.append(cur)
            start = end
        return out

    def encode(self, text: str, add_special: bool = True) -> list[int]:
        ids = [i for w in self._basic(text) for i in self._pieces(w)]
        if add_special and self.cls_id is not None and self.sep_id is not None:
            return [self.cls_id] + ids + [self.sep_id]
        return ids

    def decode(self, ids) -> str:
        out = []
        for i in ids:
            t = self.vocab[i] if 0 <= i < len(self.vocab) else ""
            if t in ("[CLS]", "[SEP]", "[PAD]"):
                continue
            if t.startswith("##") and out:
                out[-1] += t[2:]
            else:
                out.append(t)
        return " ".join(out)


class ClipTokenizer:
    """CLIP's lower-cased byte-level BPE with an end-of-word marker (``</w>``): text is cleaned,
    split by CLIP's pattern, each word's bytes are mapped to printable code points, the last symbol
    gets the marker and merges are applied by rank. Sequences are framed by <|startoftext|> /
    <|endoftext|> and optionally padded to the context length.

    Reads ``vocab.json`` + ``merges.txt`` or a ``tokenizer.json`` with the same content.
    Reference: src/HartsyInference.ModelAssets/Tokenizers/ (CLIP tokenizer)."""

    PATTERN = r"<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[\p{L}]+|[\p{N}]|[^\s\p{L}\p{N}]+"

    def __init__(self, vocab: dict[str, int], merges: Sequence[tuple[str, str]], max_len: int = 77,
                 bos: str = "<|startoftext|>", eos: str = "<|endoftext|>"):
        self.vocab = dict(vocab)
        self.inv = {i: t for t, i in self.vocab.items()}
        self.ranks = {tuple(m): r for r, m in enumerate(merges)}
        self.max_len = max_len
        self.bos_id, self.eos_id = self.vocab[bos], self.vocab[eos]
        self._b2u = _bytes_to_unicode()
        self._u2b = {u: b for b, u in self._b2u.items()}
        self._re = _re.compile(self.PATTERN, _re.IGNORECASE)
        self._cache: dict[str, list[int]] = {}

    @staticmethod
    def from_dir(path, max_len: int = 77) -> "ClipTokenizer":
        p = Path(path)
        if (p / "vocab.json").exists() and (p / "merges.txt").exists():
            vocab = json.loads((p / "vocab.json").read_text(encoding="utf-8"))
            lines = (p / "merges.txt").read_text(encoding="utf-8").split("\n")
            merges = [tuple(ln.split()) for ln in lines if ln and not ln.startswith("#version") and len(ln.split()) == 2]
        else:
            model = json.loads((p / "tokenizer.json").read_text(encoding="utf-8"))["model"]
            vocab = model["vocab"]
            merges = [tuple(m.split(" ")) if isinstance(m, str) else tuple(m) for m in model["merges"]]
        return ClipTokenizer(vocab, merges, max_len)

    def _bpe(self, word: str) -> list[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        sym = [self._b2u[b] for b in word.encode("utf-8")]
        sym[-1] += "</w>"
        while len(sym) > 1:
            best, at = None, -1
            for i in range(len(sym) - 1):
                r = self.ranks.get((sym[i], sym[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = sym[at], sym[at + 1]
            out, i = [], 0
            while i < len(sym):            # merge every occurrence of the best pair, left to right
                if i < len(sym) - 1 and sym[i] == a and sym[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(sym[i])
                    i += 1
            sym = out
        unk = self.eos_id
        ids = [self.vocab.get(s, unk) for s in sym]
        self._cache[word] = ids
        return ids

    def encode(self, text: str, add_special: bool = True, pad: bool = False) -> list[int]:
        text = " ".join(text.split()).strip().lower()
        ids: list[int] = []
        for w in self._re.findall(text):
            if w == "<|startoftext|>":
                ids.append(self.bos_id)
            elif w == "<|endoftext|>":
                ids.append(self.eos_id)
            else:
                ids += self._bpe(w)
        if add_special:
            ids = [self.bos_id] + ids[: self.max_len - 2] + [self.eos_id]
        if pad:
            ids += [self.eos_id] * (self.max_len - len(ids))
        return ids[: self.max_len]

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        out = bytearray()
        for i in ids:
            if skip_special and i in (self.bos_id, self.eos_id):
                continue
            t = self.inv.get(int(i), "")
            end = t.endswith("</w>")
            out += bytes(self._u2b[c] for c in (t[:-4] if end else t) if c in self._u2b)
            if end:
                out += b" "
        return out.decode("utf-8", errors="replace").strip()


class UnigramTokenizer:
    """SentencePiece unigram model (T5 / umT5 / XLM-R style ``tokenizer.json`` with
    ``model.type == "Unigram"``): the text is whitespace-normalised, spaces become U+2581 (with one
    in front), and the most probable segmentation into vocabulary pieces is found by a Viterbi pass
    over piece log-probabilities; characters no piece covers become the unknown id (merged when
    adjacent). ``</s>`` is appended.

    Reference: src/HartsyInference.ModelAssets/Tokenizers/ (SentencePiece unigram for T5)."""

    SPACE = "▁"

    def __init__(self, pieces: Sequence[tuple[str, float]], unk_id: int = 2, eos_id: Optional[int] = 1, add_prefix_space: bool = True,
                 specials: Optional[dict[str, int]] = None):
        self.pieces = [p for p, _ in pieces]
        self.scores = [float(s) for _, s in pieces]
        self.index = {p: i for i, p in enumerate(self.pieces)}
        self.unk_id, self.eos_id, self.add_prefix_space = unk_id, eos_id, add_prefix_space
        self.max_len = max((len(p) for p in self.pieces), default=1)
        self.specials = dict(specials or {})
        self.special_ids = set(self.specials.values())
        # an unknown character costs more than any real piece, so known pieces always win
        self.unk_score = min(self.scores, default=0.0) - 10.0

    @staticmethod
    def from_hf_json(path) -> "UnigramTokenizer":
        data = json.loads(Path(path).read_text(encoding="utf-8"))
        model = data["model"]
        if model.get("type") != "Unigram":
            raise ValueError("not a Unigram tokenizer.json")
        specials = {a["content"]: a["id"] for a in data.get("added_tokens") or [] if a.get("special")}
        eos = specials.get("</s>")
        return UnigramTokenizer([(p, s) for p, s in model["vocab"]], unk_id=model.get("unk_id") or 0, eos_id=eos, specials=specials)

    def _segment(self, text: str) -> list[int]:
        n = len(text)
        best = [float("-inf")] * (n + 1)
        back: list[tuple[int, int]] = [(0, 0)] * (n + 1)
        best[0] = 0.0
        for i in range(n):
            if best[i] == float("-inf"):
                continue
            for ln in range(1, min(self.max_len, n - i) + 1):
                pid = self.index.get(text[i:i + ln])
                if pid is None or pid in self.special_ids:
                    continue
                sc = best[i] + self.scores[pid]
                if sc > best[i + ln]:
                    best[i + ln], back[i + ln] = sc, (i, pid)
            sc = best[i] + self.unk_score
            if sc > best[i + 1]:
                best[i + 1], back[i + 1] = sc, (i, self.unk_id)
        ids: list[int] = []
        pos = n
        while pos > 0:
            prev, pid = back[pos]
            ids.append(pid)
            pos = prev
        ids.reverse()
        out: list[int] = []
        for t in ids:                              # runs of unknown characters collapse into one id
            if t == self.unk_id and out and out[-1] == self.unk_id:
                continue
            out.append(t)
        return out

    def encode(self, text: str, add_special: bool = True) -> list[int]:
        text = " ".join(text.split())
        ids: list[int] = []
        if text:
            s = text.replace(" ", self.SPACE)
            if self.add_prefix_space:
                s = self.SPACE + s
            ids = self._segment(s)
        if add_special and self.eos_id is not None:
            ids.append(self.eos_id)
        return ids

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        parts = [self.pieces[i] for i in ids if 0 <= i < len(self.pieces) and not (skip_special and i in self.special_ids)]
        return "".join(parts).replace(self.SPACE, " ").strip()
