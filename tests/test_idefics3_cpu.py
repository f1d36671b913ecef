"""Idefics3 / SmolVLM (models/vlm/idefics3.py) against ``transformers.Idefics3ForConditionalGeneration``
with random tiny weights: connector rows, logits of a prompt with one tiled picture, and the prompt
structure / image splitting rules."""
import json

import torch

from hartsyinference_b200.models.llm.config import from_hf_config
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.models.vlm.idefics3 import Idefics3Model, idefics3_vision_from_hf

IMG = 290


def _pair(vision_width: int = 32):
    from transformers import Idefics3Config, Idefics3ForConditionalGeneration
    torch.manual_seed(0)
    c = Idefics3Config(vision_config=dict(hidden_size=vision_width, intermediate_size=2 * vision_width, num_hidden_layers=2,
                                          num_attention_heads=2, image_size=32, patch_size=8),
                       text_config=dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, vocab_size=300, head_dim=16,
                                        tie_word_embeddings=False),
                       scale_factor=2, image_token_id=IMG)
    hf = Idefics3ForConditionalGeneration(c).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    text = dict(c.text_config.to_dict(), model_type="llama")
    dec = DecoderModel(from_hf_config(text), "cpu")
    dec.load_state_dict(lambda n: sd.get("model.text_model." + n[len("model."):]) if n.startswith("model.") else sd.get(n))
    mine = Idefics3Model(dec, idefics3_vision_from_hf(c.vision_config.to_dict()), IMG, 2, get=sd.get)
    return c, hf, dec, mine


def test_image_rows_and_logits_match_transformers():
    c, hf, dec, mine = _pair()
    assert mine.rows_per_tile == 4
    views = torch.randn(3, 3, 32, 32)                       # two tiles and the global view, already normalised
    with torch.no_grad():
        want = hf.model.get_image_features(views[None])
    want = getattr(want, "pooler_output", want)
    want = torch.cat(list(want)) if isinstance(want, (list, tuple)) else want.reshape(-1, want.shape[-1])
    got = mine.view_features(views).float()
    assert got.shape == want.shape == (12, 64)
    assert torch.nn.functional.cosine_similarity(got, want, dim=-1).min() > 0.999
    # a prompt with the three views in place: logits of the mixed sequence
    ids = [5, 6] + [IMG] * 4 + [7] + [IMG] * 4 + [8, 9] + [IMG] * 4 + [10, 11]
    with torch.no_grad():
        ref = hf(input_ids=torch.tensor([ids]), pixel_values=views[None]).logits[0]
    t = len(ids)
    emb = dec.embed[torch.tensor(ids)].clone()
    emb[torch.tensor(ids) == IMG] = mine.view_features(views).to(emb.dtype)
    dec.alloc_kv(4, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(t, dtype=torch.int32),
                     slot_mapping=torch.arange(t, dtype=torch.int64), block_table=torch.arange(4, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([t], dtype=torch.int32), is_decode=False, cu_q=torch.tensor([0, t], dtype=torch.int32),
                     max_q_len=t, max_kv_len=t, embeds=emb)
    out = dec.full_logits(dec.forward_hidden(b)).float()
    assert torch.nn.functional.cosine_similarity(out, ref, dim=-1).min() > 0.995


def test_splitting_and_prompt_structure():
    _, _, _, mine = _pair()
    mine.longest_edge = 64
    views, r, c = mine.split_image(torch.rand(3, 40, 80))          # 32 x 64 after the resize: one row of two tiles
    assert (r, c) == (1, 2) and views.shape == (3, 3, 32, 32) and float(views.min()) >= -1 and float(views.max()) <= 1
    small, r0, c0 = mine.split_image(torch.rand(3, 10, 12))
    mine.longest_edge = 32
    one, r1, c1 = mine.split_image(torch.rand(3, 10, 12))
    assert (r1, c1) == (0, 0) and one.shape == (1, 3, 32, 32)
    names = {"<fake_token_around_image>": 280, "<global-img>": 281, "<row_1_col_1>": 282, "<row_1_col_2>": 283}
    mine.bind_tokenizer(names.get, [13])
    img = [IMG] * 4
    assert mine.image_block(1, 2) == [280, 282] + img + [280, 283] + img + [13, 13, 280, 281] + img + [280]
    assert mine.image_block(0, 0) == [280, 281] + img + [280]
    mine.longest_edge = 64
    ids, emb, mask = mine.expand_prompt([5, IMG, 6], [torch.rand(3, 40, 80)])
    assert ids[0] == 5 and ids[-1] == 6 and ids[1:-1] == mine.image_block(1, 2)
    assert emb.shape == (len(ids), 64) and int(mask.sum()) == 12 and bool((emb[~mask] == 0).all())


def test_loader_builds_the_model_from_a_checkpoint_directory(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.models.llm.loader import load_llm
    c, hf, _, _ = _pair()
    d = tmp_path / "smol"
    d.mkdir()
    cfg = c.to_dict()
    cfg["model_type"] = "idefics3"
    (d / "config.json").write_text(json.dumps(cfg))
    (d / "preprocessor_config.json").write_text(json.dumps({"size": {"longest_edge": 64}}))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, d / "model.safetensors")
    llm = load_llm(str(d), "cpu")
    assert llm.vlm is not None and llm.vlm.longest_edge == 64 and llm.vlm.rows_per_tile == 4
    ids, emb, mask = llm.vlm.expand_prompt([3, IMG, 4], [torch.rand(3, 20, 40)])
    assert int(mask.sum()) == 12 and emb.shape[0] == len(ids)


import pytest


@pytest.mark.gpu
def test_gpu_image_rows_agree_with_cpu():
    c, hf, _, mine = _pair(vision_width=128)            # head dim 64: the device attention kernel's smallest
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    text = dict(c.text_config.to_dict(), model_type="llama")
    dec = DecoderModel(from_hf_config(text), "cuda")
    dec.load_state_dict(lambda n: sd.get("model.text_model." + n[len("model."):]) if n.startswith("model.") else sd.get(n))
    gpu = Idefics3Model(dec, idefics3_vision_from_hf(c.vision_config.to_dict()), IMG, 2, get=sd.get)
    views = torch.randn(2, 3, 32, 32)
    a, b = mine.view_features(views).float(), gpu.view_features(views.cuda()).float().cpu()
    assert torch.nn.functional.cosine_similarity(a, b, dim=-1).min() > 0.99
