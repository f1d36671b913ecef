import json

import pytest

from hartsyinference_b200.assets.chat_template import ChatTemplate
from hartsyinference_b200.assets.tokenizer import ByteTokenizer, Tokenizer, _B2U


def _toy_bpe(tmp_path):
    # byte-level vocabulary: 256 bytes + a few merges, in tokenizer.json form
    vocab = {_B2U[b]: b for b in range(256)}
    merges = []

    def add(a, b):
        vocab[a + b] = len(vocab)
        merges.append(f"{a} {b}")

    sp = _B2U[ord(" ")]
    add("h", "e"); add("l", "l"); add("he", "ll"); add("hell", "o"); add(sp, "w"); add(sp + "w", "o")
    add("r", "l"); add(sp + "wo", "rl"); add(sp + "worl", "d")
    tj = {"model": {"type": "BPE", "vocab": vocab, "merges": merges},
          "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
          "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
          "added_tokens": [{"id": len(vocab), "content": "<|eot|>", "single_word": False, "lstrip": False,
                            "rstrip": False, "normalized": False, "special": True}]}
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(tj), encoding="utf-8")
    return Tokenizer.from_hf_json(p), vocab


def test_rank_bpe_merges_and_roundtrip(tmp_path):
    tok, vocab = _toy_bpe(tmp_path)
    ids = tok.encode("hello world")
    sp = _B2U[ord(" ")]
    assert ids == [vocab["hello"], vocab[sp + "world"]]
    text = "hello world ✓ naïve\n\tüber<|eot|>x"
    ids = tok.encode(text)
    assert tok.special_tokens["<|eot|>"] in ids
    assert tok.decode(ids, skip_special=False) == text
    assert tok.decode(ids) == text.replace("<|eot|>", "")


def test_stream_decoder_never_emits_broken_utf8(tmp_path):
    tok, _ = _toy_bpe(tmp_path)
    text = "héllo ✓✓ 日本語"
    sd = tok.stream_decoder()
    out = ""
    for t in tok.encode(text):
        piece = sd.push(t)
        assert "�" not in piece
        out += piece
    assert out + sd.flush() == text


def test_against_hf_tokenizers_if_available(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    tok, _ = _toy_bpe(tmp_path)
    ref = tokenizers.Tokenizer.from_file(str(tmp_path / "tokenizer.json"))
    for s in ("hello world", "hello  world hello", "wor ld hellohello"):
        assert tok.encode(s) == ref.encode(s).ids


def test_spm_gguf_vocab():
    tokens = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "he", "ll", "hell", "hello", "▁hello", "▁w", "▁wo"]
    types = [2, 3, 3] + [6] * 256 + [1] * 12
    scores = [0.0] * 259 + [-1.0, -2, -2, -2, -2, -3, -4, -5, -6, -7, -8, -9]
    md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.token_type": types,
          "tokenizer.ggml.scores": scores, "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    tok = Tokenizer.from_gguf_metadata(md)
    ids = tok.encode("hello wZ")
    assert ids[0] == 1 and ids[1] == tokens.index("▁hello")
    assert tok.decode(ids) == "hello wZ"       # 'Z' went through the byte-fallback tokens
    assert tokens.index("<0x5A>") in ids


def test_byte_tokenizer_and_chat_template():
    bt = ByteTokenizer({"<eos>": 256}, vocab_size=300)
    ids = bt.encode("hi<eos>")
    assert ids == [104, 105, 256] and bt.decode(ids) == "hi"
    ct = ChatTemplate("chatml")
    s = ct.render([{"role": "system", "content": "S"}, {"role": "user", "content": "U"}])
    assert s == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n<|im_start|>assistant\n"
    l3 = ChatTemplate.for_arch("llama").render([{"role": "user", "content": " hi "}])
    assert l3.startswith("<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>")
    with pytest.raises(Exception):
        ChatTemplate("{{ raise_exception('no') }}").render([])


def test_unigram_tokenizer_matches_the_tokenizers_library(tmp_path):
    import pytest
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer as HfTok, decoders, models, normalizers, pre_tokenizers, processors
    from hartsyinference_b200.assets.tokenizer import UnigramTokenizer
    sp = "▁"
    vocab = [("<pad>", 0.0), ("</s>", 0.0), ("<unk>", 0.0), (sp, -2.0), (sp + "the", -3.0), (sp + "cat", -5.0), ("s", -3.5), (sp + "sat", -6.0),
             (sp + "on", -4.5), ("a", -3.2), ("t", -3.3), ("c", -4.0), ("h", -4.1), ("e", -3.0), ("n", -3.6), ("o", -3.4), (sp + "mat", -7.0),
             ("at", -4.2), (sp + "c", -5.5), ("the", -4.8), (sp + "t", -4.4), ("m", -4.6), (".", -3.9), ("on", -4.9), ("ca", -6.5), ("ts", -6.0)]
    hf = HfTok(models.Unigram(vocab, unk_id=2))
    hf.normalizer = normalizers.Sequence([normalizers.Replace(tk.Regex(" {2,}"), " ")])
    hf.pre_tokenizer = pre_tokenizers.Metaspace(replacement=sp, prepend_scheme="always")
    hf.post_processor = processors.TemplateProcessing(single="$A </s>", special_tokens=[("</s>", 1)])
    hf.decoder = decoders.Metaspace(replacement=sp, prepend_scheme="always")
    hf.add_special_tokens(["<pad>", "</s>", "<unk>"])
    hf.save(str(tmp_path / "tokenizer.json"))
    mine = UnigramTokenizer.from_hf_json(tmp_path / "tokenizer.json")
    for text in ["the cat sat on the mat.", "cats", "the  cats   on a mat", "that", "the zebra", ""]:
        assert mine.encode(text) == hf.encode(text).ids, text
    assert mine.decode(mine.encode("the cat sat")) == "the cat sat"
