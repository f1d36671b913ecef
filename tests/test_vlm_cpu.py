"""Vision tower parity against transformers' CLIPVisionModel, and LLaVA-style generation through
the serving engine with image embeddings spliced into the prompt."""
import pytest
import torch

from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.encoders.clip_vision import ClipVisionEncoder, preprocess_image, tiny_clip_vision
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel
from hartsyinference_b200.models.vlm import LlavaModel


def test_clip_vision_matches_transformers():
    tr = pytest.importorskip("transformers")
    cfg = tiny_clip_vision()
    hf_cfg = tr.CLIPVisionConfig(hidden_size=cfg.width, intermediate_size=cfg.width * cfg.mlp_ratio,
                                 num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                                 image_size=cfg.image_size, patch_size=cfg.patch, hidden_act="quick_gelu")
    torch.manual_seed(0)
    hf = tr.CLIPVisionModel(hf_cfg).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    enc = ClipVisionEncoder(cfg, "cpu", get=lambda n: sd.get(n))
    img = torch.randn(3, cfg.image_size, cfg.image_size)
    with torch.no_grad():
        out = hf(pixel_values=img[None], output_hidden_states=True)
    mine = enc.hidden_states(img, -2).float()
    ref = out.hidden_states[-2][0]
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.995
    pooled = enc.embed(img).float()
    assert torch.nn.functional.cosine_similarity(pooled, out.pooler_output[0], dim=0) > 0.995


def _toy():
    m = DecoderModel(C.tiny(), "cpu")
    m.random_init(3, std=0.05)
    return m


def test_llava_generate_uses_image_embeddings():
    model = _toy()
    image_tok = model.cfg.vocab_size - 1
    vcfg = tiny_clip_vision()
    vlm = LlavaModel(model, vcfg, image_tok, seed=5)
    img_a = torch.randn(3, 32, 32, generator=torch.Generator().manual_seed(1))
    img_b = torch.randn(3, 32, 32, generator=torch.Generator().manual_seed(2)) * 3
    prompt = [5, 9, image_tok, 11, 12]
    ids, embeds, mask = vlm.expand_prompt(prompt, [img_a])
    n = vcfg.num_patches
    assert len(ids) == len(prompt) - 1 + n and int(mask.sum()) == n
    assert mask.tolist() == [False, False] + [True] * n + [False, False]

    # what reaches the decoder: token embeddings, with the image rows replaced by projected patches
    seen = []
    inner = model.forward_hidden

    def spy(batch, *a, **k):
        if batch.embeds is not None:
            seen.append(batch.embeds.clone())
        return inner(batch, *a, **k)

    model.forward_hidden = spy
    params = SamplingParams(greedy=True, max_tokens=4)
    chunked = LLMEngine(model, num_pages=64, page_size=4, max_batch=2, prefill_chunk=8, max_model_len=64)
    out_chunked = vlm.generate(chunked, prompt, [img_a], params)
    got = torch.cat(seen, 0)
    want = model.embed[torch.tensor(ids)].clone()
    want[mask] = embeds[mask]
    assert len(seen) > 1 and torch.equal(got, want)
    model.forward_hidden = inner

    # chunked prefill of the mixed embeddings gives the same tokens as one whole-prompt prefill
    whole = LLMEngine(model, num_pages=64, page_size=4, max_batch=2, prefill_chunk=256, max_model_len=64)
    out_whole = vlm.generate(whole, prompt, [img_a], params)
    assert len(out_chunked) == 4 and out_chunked == out_whole

    # a different image changes the patch embeddings
    _, embeds_b, _ = vlm.expand_prompt(prompt, [img_b])
    assert not torch.allclose(embeds_b[mask].float(), embeds[mask].float())
    with pytest.raises(ValueError):
        vlm.expand_prompt(prompt, [])
    with pytest.raises(ValueError):
        vlm.expand_prompt(prompt, [img_a, img_b])


def _llava_checkpoint(tmp_path, layout: str):
    """A tiny LLaVA checkpoint directory in one of the two tensor-name layouts."""
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    tr = pytest.importorskip("transformers")
    vc = tiny_clip_vision()
    torch.manual_seed(1)
    hf_v = tr.CLIPVisionModel(tr.CLIPVisionConfig(hidden_size=vc.width, intermediate_size=vc.width * vc.mlp_ratio,
                                                  num_hidden_layers=vc.layers, num_attention_heads=vc.heads,
                                                  image_size=vc.image_size, patch_size=vc.patch))
    lcfg = tr.LlamaConfig(vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256,
                          tie_word_embeddings=False)
    hf_l = tr.LlamaForCausalLM(lcfg)
    H = lcfg.hidden_size
    proj = {"multi_modal_projector.linear_1.weight": torch.randn(H, vc.width) * 0.05,
            "multi_modal_projector.linear_1.bias": torch.zeros(H),
            "multi_modal_projector.linear_2.weight": torch.randn(H, H) * 0.05,
            "multi_modal_projector.linear_2.bias": torch.zeros(H)}
    tensors = {}
    for k, v in hf_l.state_dict().items():
        if layout == "old":
            tensors["language_model." + k] = v
        else:
            tensors[("model.language_model." + k[len("model."):]) if k.startswith("model.") else k] = v
    for k, v in list(hf_v.state_dict().items()) + list(proj.items()):
        k = k if k.startswith("multi_modal") else "vision_tower." + k
        tensors[k if layout == "old" else "model." + k] = v
    tensors = {k: v.detach().to(torch.bfloat16).contiguous() for k, v in tensors.items()}
    cfg = {"model_type": "llava", "image_token_index": 299, "vision_feature_layer": -2,
           "text_config": {**lcfg.to_dict(), "model_type": "llama"},
           "vision_config": {"hidden_size": vc.width, "intermediate_size": vc.width * vc.mlp_ratio,
                             "num_hidden_layers": vc.layers, "num_attention_heads": vc.heads,
                             "image_size": vc.image_size, "patch_size": vc.patch, "hidden_act": "quick_gelu"}}
    d = tmp_path / f"llava-{layout}"
    save_hf_checkpoint(cfg, tensors, d)
    return d


@pytest.mark.parametrize("layout", ["old", "new"])
def test_llava_checkpoint_through_text_service(tmp_path, layout):
    import numpy as np
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, TextRequest
    d = _llava_checkpoint(tmp_path, layout)
    eng = InferenceEngine("cpu")
    try:
        spec = ModelSpec(str(d))
        img = (np.random.default_rng(0).random((40, 52, 3)) * 255).astype(np.uint8)
        req = TextRequest(prompt="look: <image> what is it?", images=[img], max_tokens=3, greedy=True)
        res = eng.text.generate(spec, req)
        assert len(res.token_ids) == 3 and res.error is None
        n = tiny_clip_vision().num_patches
        plain = eng.text.generate(spec, TextRequest(prompt="look: <image> what is it?", max_tokens=3, greedy=True))
        assert res.prompt_tokens > n                      # the image token expanded to its patches
        assert plain.prompt_tokens < res.prompt_tokens    # without images "<image>" is ordinary text
        other = (np.random.default_rng(1).random((40, 52, 3)) * 255).astype(np.uint8)
        h = eng.text._host(spec)
        a = h.llm.vlm.image_features(preprocess_image(img, 32))
        b = h.llm.vlm.image_features(preprocess_image(other, 32))
        assert a.shape == (n, 128) and not torch.allclose(a.float(), b.float())
    finally:
        eng.text.release()


def test_server_flattens_openai_image_parts():
    import base64
    import io
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (8, 8), (255, 0, 0)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    from hartsyinference_b200.server.app import _flatten_parts
    msgs, images = _flatten_parts([{"role": "user", "content": [{"type": "text", "text": "hi "},
                                                                      {"type": "image_url", "image_url": {"url": url}}]},
                                         {"role": "system", "content": "plain"}])
    assert msgs[0]["content"] == "hi <image>\n" and msgs[1]["content"] == "plain"
    assert len(images) == 1 and images[0].size == (8, 8)
    with pytest.raises(ValueError):
        _flatten_parts([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}])


def _clip_dir(tmp_path):
    """A tiny two-tower CLIP checkpoint with a byte-level vocab.json / merges.txt."""
    import json
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    tr = pytest.importorskip("transformers")
    b2u = _bytes_to_unicode()
    vocab = {}
    for b in range(256):
        vocab[b2u[b]] = len(vocab)
    for b in range(256):
        vocab[b2u[b] + "</w>"] = len(vocab)
    merges = [("c", "a"), ("ca", "t</w>"), ("d", "o"), ("do", "g</w>"), ("a</w>", "x")]
    for a, b in merges[:4]:
        vocab[a + b] = len(vocab)
    vocab["<|startoftext|>"] = len(vocab)
    vocab["<|endoftext|>"] = len(vocab)
    vc = tiny_clip_vision()
    cfg = tr.CLIPConfig(
        text_config=dict(vocab_size=len(vocab), hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                         max_position_embeddings=16, bos_token_id=vocab["<|startoftext|>"], eos_token_id=vocab["<|endoftext|>"],
                         pad_token_id=vocab["<|endoftext|>"]),
        vision_config=dict(hidden_size=vc.width, intermediate_size=vc.width * vc.mlp_ratio, num_hidden_layers=vc.layers,
                           num_attention_heads=vc.heads, image_size=vc.image_size, patch_size=vc.patch),
        projection_dim=32)
    torch.manual_seed(2)
    hf = tr.CLIPModel(cfg).eval()
    d = tmp_path / "clip-synth"
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()
                                       if "position_ids" not in k}, d)
    (d / "vocab.json").write_text(json.dumps(vocab))
    (d / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges[:4]) + "\n")
    return d, hf, tr.CLIPTokenizer(str(d / "vocab.json"), str(d / "merges.txt"))


def test_clip_tokenizer_and_vision_service(tmp_path):
    from hartsyinference_b200.assets.tokenizer import ClipTokenizer
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, VisionRequest
    d, hf, hf_tok = _clip_dir(tmp_path)
    tok = ClipTokenizer.from_dir(d, max_len=77)
    for text in ["A cat", "the DOG, and a cat!", "naïve café 日本", ""]:
        assert tok.encode(text) == hf_tok(text)["input_ids"]
    tok = ClipTokenizer.from_dir(d, max_len=16)
    long = tok.encode("the dog and the cat and the dog again")
    assert len(long) == 16 and long[0] == tok.bos_id and long[-1] == tok.eos_id
    assert tok.decode(tok.encode("a cat and dog")) == "a cat and dog"
    assert len(tok.encode("x", pad=True)) == 16

    eng = InferenceEngine("cpu")
    rng = torch.Generator().manual_seed(0)
    imgs = [torch.rand(3, 32, 32, generator=rng), torch.rand(3, 32, 32, generator=rng)]
    texts = ["a cat", "a dog and a cat"]
    res = eng.vision.run(ModelSpec(str(d)), VisionRequest(images=imgs, texts=texts))
    assert res.image_embeddings.shape == (2, 32) and res.text_embeddings.shape == (2, 32) and res.similarity.shape == (2, 2)
    with torch.no_grad():
        px = torch.stack([preprocess_image(im, 32) for im in imgs])
        fi = hf.get_image_features(pixel_values=px)
        enc = hf_tok(texts, padding=True, return_tensors="pt")
        ft = hf.get_text_features(**enc)
    fi = getattr(fi, "pooler_output", fi)
    ft = getattr(ft, "pooler_output", ft)
    fi, ft = fi / fi.norm(dim=-1, keepdim=True), ft / ft.norm(dim=-1, keepdim=True)
    assert torch.nn.functional.cosine_similarity(res.image_embeddings.flatten(), fi.flatten(), dim=0) > 0.99
    assert torch.nn.functional.cosine_similarity(res.text_embeddings.flatten(), ft.flatten(), dim=0) > 0.99
    assert (res.similarity - fi @ ft.t()).abs().max() < 0.05
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="detect", images=imgs))
    eng.close()


@pytest.mark.parametrize("kind", ["siglip", "dinov2"])
def test_vit_embedders_match_transformers(kind):
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.encoders.vit import VitEncoder, tiny_vit, vit_from_hf
    cfg = tiny_vit(kind)
    torch.manual_seed(0)
    if kind == "siglip":
        hc = tr.SiglipVisionConfig(hidden_size=cfg.width, intermediate_size=cfg.ffn, num_hidden_layers=cfg.layers,
                                   num_attention_heads=cfg.heads, image_size=cfg.image_size, patch_size=cfg.patch)
        hf = tr.SiglipVisionModel(hc).eval()
    else:
        hc = tr.Dinov2Config(hidden_size=cfg.width, mlp_ratio=cfg.ffn // cfg.width, num_hidden_layers=cfg.layers,
                             num_attention_heads=cfg.heads, image_size=cfg.image_size, patch_size=cfg.patch)
        hf = tr.Dinov2Model(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "embeddings" not in n:
                p.mul_(2.0)
            if "lambda1" in n:
                p.copy_(0.5 + torch.rand_like(p))
    assert vit_from_hf(hc.to_dict()) == cfg
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    enc = VitEncoder(cfg, "cpu", get=lambda n: sd.get(n))
    img = torch.randn(3, cfg.image_size, cfg.image_size, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        out = hf(pixel_values=img[None])
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0)
    assert cos(enc.hidden_states(img), out.last_hidden_state[0]) > 0.995
    assert cos(enc.embed(img), out.pooler_output[0]) > 0.995
    if kind == "dinov2":
        assert enc.embed(img, concat_patch_mean=True).shape == (2 * cfg.width,)


def test_vision_service_loads_dinov2(tmp_path):
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, VisionRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    hc = tr.Dinov2Config(hidden_size=128, mlp_ratio=2, num_hidden_layers=2, num_attention_heads=2, image_size=32, patch_size=8)
    torch.manual_seed(0)
    hf = tr.Dinov2Model(hc).eval()
    save_hf_checkpoint(hc.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, tmp_path / "dino")
    eng = InferenceEngine("cpu")
    imgs = [torch.rand(3, 40, 40, generator=torch.Generator().manual_seed(i)) for i in range(2)]
    res = eng.vision.run(ModelSpec(str(tmp_path / "dino")), VisionRequest(images=imgs))
    assert res.image_embeddings.shape == (2, 128) and res.text_embeddings is None
    assert torch.allclose(res.image_embeddings.norm(dim=-1), torch.ones(2), atol=1e-3)
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(tmp_path / "dino")), VisionRequest(texts=["a"]))
    eng.close()


def test_depth_anything_matches_transformers_and_serves(tmp_path):
    tr = pytest.importorskip("transformers")
    import base64
    import io
    from fastapi.testclient import TestClient
    from PIL import Image
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, VisionRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    from hartsyinference_b200.models.vision.depth_anything import DepthAnything, depth_anything_from_hf
    from hartsyinference_b200.server.app import ServerOptions, create_app
    bc = tr.Dinov2Config(hidden_size=128, num_hidden_layers=4, num_attention_heads=2, image_size=28, patch_size=14, mlp_ratio=2,
                         out_indices=[1, 2, 3, 4], reshape_hidden_states=False, apply_layernorm=True)
    c = tr.DepthAnythingConfig(backbone_config=bc, reassemble_hidden_size=128, neck_hidden_sizes=[16, 32, 64, 64],
                               fusion_hidden_size=32, head_hidden_size=16, patch_size=14, reassemble_factors=[4, 2, 1, 0.5])
    torch.manual_seed(0)
    hf = tr.DepthAnythingForDepthEstimation(c).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "embeddings" not in n:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = DepthAnything(depth_anything_from_hf(c.to_dict()), "cpu", get=lambda n: sd.get(n))
    for hw in ((28, 28), (42, 56)):          # the second size resamples the position table
        img = torch.randn(3, *hw, generator=torch.Generator().manual_seed(1))
        with torch.no_grad():
            ref = hf(pixel_values=img[None]).predicted_depth[0]
        mine = m.predict(img)
        assert mine.shape == ref.shape
        assert torch.nn.functional.cosine_similarity(ref.flatten(), mine.flatten(), dim=0) > 0.999

    d = tmp_path / "depth"
    save_hf_checkpoint(c.to_dict(), {k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, d)
    eng = InferenceEngine("cpu")
    pic = (torch.rand(30, 45, 3, generator=torch.Generator().manual_seed(2)) * 255).to(torch.uint8)
    res = eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="depth", images=[pic]))
    assert len(res.depth) == 1 and res.depth[0].shape == (30, 45) and res.depth[0].min() >= 0
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="embed", images=[pic]))
    buf = io.BytesIO()
    Image.fromarray(pic.numpy()).save(buf, format="PNG")
    with TestClient(create_app(ServerOptions(models={"depth": str(d)}), engine=eng)) as cl:
        r = cl.post("/v1/native/vision", json={"model": "depth", "operation": "depth", "images": [base64.b64encode(buf.getvalue()).decode()]})
        assert r.status_code == 200, r.text
        j = r.json()["depth"][0]
        assert (j["width"], j["height"]) == (45, 30)
        assert Image.open(io.BytesIO(base64.b64decode(j["png16_base64"]))).size == (45, 30)
    eng.close()


def test_llava_next_anyres_matches_transformers():
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.vlm.llava_next import LlavaNextModel, select_best_resolution
    vc = tiny_clip_vision()                       # 32 x 32 input, 8 x 8 patches -> 16 patch tokens per view
    pins = [(32, 64), (64, 32), (64, 64), (96, 32), (32, 96)]
    hv = tr.CLIPVisionConfig(hidden_size=vc.width, intermediate_size=vc.width * vc.mlp_ratio, num_hidden_layers=vc.layers,
                             num_attention_heads=vc.heads, image_size=vc.image_size, patch_size=vc.patch)
    ht = tr.LlamaConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                        num_key_value_heads=2, max_position_embeddings=512)
    cfg = tr.LlavaNextConfig(vision_config=hv, text_config=ht, image_grid_pinpoints=[list(p) for p in pins], image_token_index=319,
                             vision_feature_layer=-2, vision_feature_select_strategy="default")
    torch.manual_seed(0)
    hf = tr.LlavaNextForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        hf.model.image_newline.copy_(torch.randn(128) * 0.1)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}

    def get(name):      # this transformers version nests everything under "model."
        for cand in (name, "model." + name):
            if cand in sd:
                return sd[cand]
        return None
    dec = DecoderModel(C.tiny(vocab_size=320, hidden_size=128, num_heads=2, num_kv_heads=2, head_dim=64), "cpu")
    dec.random_init(1)
    m = LlavaNextModel(dec, vc, 319, get=get, pinpoints=pins)
    for (h, w) in ((40, 90), (70, 50), (33, 31)):
        img = torch.rand(3, h, w, generator=torch.Generator().manual_seed(h))
        views, grid = m.tiles(img)
        best = select_best_resolution((h, w), pins)
        assert grid == (best[0] // 32, best[1] // 32) and views.shape == (1 + grid[0] * grid[1], 3, 32, 32)
        with torch.no_grad():
            ref = hf.get_image_features(pixel_values=views[None], image_sizes=torch.tensor([[h, w]]),
                                        vision_feature_layer=-2, vision_feature_select_strategy="default")
        ref = ref.pooler_output if hasattr(ref, "pooler_output") else ref
        ref = ref[0] if isinstance(ref, (list, tuple)) else ref
        mine = m.image_features_anyres(img)
        assert mine.shape == ref.shape, (mine.shape, ref.shape)
        assert torch.nn.functional.cosine_similarity(mine.float().flatten(), ref.float().flatten(), dim=0) > 0.99
    ids, embeds, mask = m.expand_prompt([5, 319, 7], [torch.rand(3, 40, 90)])
    assert int(mask.sum()) == m.image_features_anyres(torch.rand(3, 40, 90)).shape[0] and len(ids) == int(mask.sum()) + 2


def test_llava_next_checkpoint_through_text_service(tmp_path):
    import numpy as np
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, TextRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    import json
    d = _llava_checkpoint(tmp_path, "new")
    cfg = json.loads((d / "config.json").read_text())
    cfg.update(model_type="llava_next", image_grid_pinpoints=[[32, 64], [64, 32], [64, 64]])
    (d / "config.json").write_text(json.dumps(cfg))
    from hartsyinference_b200.assets.safetensors import SafeTensorsFile, save_file
    f = SafeTensorsFile(d / "model.safetensors")
    tensors = {k: f.get(k) for k in f.keys()}
    tensors["model.image_newline"] = torch.randn(128).to(torch.bfloat16)
    save_file(tensors, d / "model.safetensors")
    eng = InferenceEngine("cpu")
    try:
        wide = (np.random.default_rng(0).random((30, 80, 3)) * 255).astype(np.uint8)
        tall = (np.random.default_rng(1).random((80, 30, 3)) * 255).astype(np.uint8)
        a = eng.text.generate(ModelSpec(str(d)), TextRequest(prompt="<image> describe", images=[wide], max_tokens=2, greedy=True))
        b = eng.text.generate(ModelSpec(str(d)), TextRequest(prompt="<image> describe", images=[tall], max_tokens=2, greedy=True))
        assert len(a.token_ids) == 2 and a.error is None and b.error is None
        assert a.prompt_tokens != b.prompt_tokens           # the token count follows the image's shape
        assert type(eng.text._host(ModelSpec(str(d))).llm.vlm).__name__ == "LlavaNextModel"
    finally:
        eng.text.release()


def test_clip_text_penultimate_states_and_projection():
    """What SDXL / SD3 take from a CLIP text tower: hidden_states[-2] and the projected pooled vector."""
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.encoders.clip import ClipTextEncoder, clip_text_from_hf
    hc = tr.CLIPTextConfig(vocab_size=128, hidden_size=64, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                           max_position_embeddings=16, hidden_act="gelu", projection_dim=32, eos_token_id=127, bos_token_id=126, pad_token_id=127)
    torch.manual_seed(0)
    hf = tr.CLIPTextModelWithProjection(hc).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = clip_text_from_hf(hc.to_dict())
    assert not cfg.quick_gelu and cfg.layers == 3
    enc = ClipTextEncoder(cfg, "cpu", get=lambda n: sd.get(n))
    ids = torch.tensor([126, 5, 9, 33, 127])
    with torch.no_grad():
        out = hf(input_ids=ids[None], output_hidden_states=True)
    states, pooled = enc.encode(ids, layer=-2, project=True)
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0)
    assert cos(states, out.hidden_states[-2][0]) > 0.995
    assert pooled.shape == (32,) and cos(pooled, out.text_embeds[0]) > 0.995
    last, _ = enc.encode(ids)
    assert cos(last, out.last_hidden_state[0]) > 0.995


def test_clipseg_matches_transformers_and_serves(tmp_path):
    tr = pytest.importorskip("transformers")
    import base64
    import io
    import json
    from fastapi.testclient import TestClient
    from PIL import Image
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, VisionRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    from hartsyinference_b200.models.vision.clipseg import ClipSeg, clipseg_from_hf
    from hartsyinference_b200.server.app import ServerOptions, create_app
    b2u = _bytes_to_unicode()
    vocab = {}
    for b in range(256):
        vocab[b2u[b]] = len(vocab)
    for b in range(256):
        vocab[b2u[b] + "</w>"] = len(vocab)
    vocab["<|startoftext|>"], vocab["<|endoftext|>"] = len(vocab), len(vocab) + 1
    vc = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=2, image_size=32, patch_size=8)
    tc = dict(vocab_size=len(vocab), hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
              max_position_embeddings=16, eos_token_id=len(vocab) - 1, bos_token_id=len(vocab) - 2, pad_token_id=len(vocab) - 1)
    c = tr.CLIPSegConfig(text_config=tc, vision_config=vc, projection_dim=32, extract_layers=[1, 2, 3], reduce_dim=16,
                         decoder_num_attention_heads=2, decoder_intermediate_size=32, conditional_layer=0)
    torch.manual_seed(0)
    hf = tr.CLIPSegForImageSegmentation(c).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "embed" not in n:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = ClipSeg(clipseg_from_hf(c.to_dict()), "cpu", get=lambda n: sd.get(n))
    img = torch.randn(3, 32, 32, generator=torch.Generator().manual_seed(1))
    ids = torch.tensor([len(vocab) - 2, 5, 7, len(vocab) - 1])
    with torch.no_grad():
        ref = hf(pixel_values=img[None], input_ids=ids[None]).logits[0]
    mine = m.segment(img, m.text_embedding(ids))
    assert mine.shape == ref.shape == (32, 32)
    assert torch.nn.functional.cosine_similarity(ref.flatten(), mine.flatten(), dim=0) > 0.995

    d = tmp_path / "clipseg"
    save_hf_checkpoint(c.to_dict(), {k: v.contiguous() for k, v in sd.items() if "position_ids" not in k}, d)
    (d / "vocab.json").write_text(json.dumps(vocab))
    (d / "merges.txt").write_text("#version: 0.2\n")
    eng = InferenceEngine("cpu")
    pic = (torch.rand(40, 56, 3, generator=torch.Generator().manual_seed(2)) * 255).to(torch.uint8)
    res = eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="segment", images=[pic], texts=["a cat", "the sky"]))
    assert len(res.masks) == 1 and res.masks[0].shape == (2, 40, 56) and 0 <= float(res.masks[0].min()) and float(res.masks[0].max()) <= 1
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="segment", images=[pic]))
    buf = io.BytesIO()
    Image.fromarray(pic.numpy()).save(buf, format="PNG")
    with TestClient(create_app(ServerOptions(models={"seg": str(d)}), engine=eng)) as cl:
        r = cl.post("/v1/native/vision", json={"model": "seg", "operation": "segment", "texts": ["a cat"],
                                               "images": [base64.b64encode(buf.getvalue()).decode()]})
        assert r.status_code == 200, r.text
        mk = r.json()["masks"][0][0]
        assert (mk["width"], mk["height"]) == (56, 40) and 0 <= mk["coverage"] <= 1
    eng.close()


def _owlvit_pair():
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.vision.owlvit import OwlVit, owlvit_from_hf
    vc = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2, image_size=32, patch_size=8)
    tc = dict(vocab_size=514, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
              max_position_embeddings=16, eos_token_id=513, bos_token_id=512, pad_token_id=0)
    c = tr.OwlViTConfig(text_config=tc, vision_config=vc, projection_dim=64)
    torch.manual_seed(0)
    hf = tr.OwlViTForObjectDetection(c).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "encoder.layers" in n:
                p.mul_(2.0)
            if n.startswith("box_head") and p.ndim == 2:
                p.mul_(4.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    return c, hf, sd, OwlVit(owlvit_from_hf(c.to_dict()), "cpu", get=lambda n: sd.get(n))


def test_owlvit_matches_transformers():
    from hartsyinference_b200.models.vision.owlvit import OwlVit
    c, hf, sd, m = _owlvit_pair()
    img = torch.randn(3, 32, 32, generator=torch.Generator().manual_seed(1))
    ids = torch.tensor([[512, 5, 7, 513], [512, 9, 513, 0]])
    with torch.no_grad():
        ref = hf(pixel_values=img[None], input_ids=ids, attention_mask=(ids != 0).long())
    q = torch.stack([m.text_embedding(ids[0]), m.text_embedding(ids[1][:3])])
    logits, boxes = m.detect(img, q)
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0)
    assert logits.shape == (16, 2) and cos(ref.logits[0], logits) > 0.995
    assert boxes.shape == (16, 4) and (ref.pred_boxes[0] - boxes).abs().max() < 0.02
    assert torch.equal(OwlVit.box_bias(4, 4), hf.compute_box_bias(4, 4))


def test_detect_operation_and_nms(tmp_path):
    import json
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, VisionRequest
    from hartsyinference_b200.engine.vision_service import nms
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    boxes = torch.tensor([[0, 0, 10, 10], [1, 1, 11, 11], [20, 20, 30, 30], [0, 0, 10, 9.0]])
    assert nms(boxes, torch.tensor([0.9, 0.8, 0.7, 0.95]), 0.5) == [3, 2]
    assert nms(boxes, torch.tensor([0.9, 0.8, 0.7, 0.95]), 0.95) == [3, 0, 1, 2]
    c, hf, sd, _ = _owlvit_pair()
    b2u = _bytes_to_unicode()
    vocab = {}
    for b in range(256):
        vocab[b2u[b]] = len(vocab)
    for b in range(256):
        vocab[b2u[b] + "</w>"] = len(vocab)
    vocab["<|startoftext|>"], vocab["<|endoftext|>"] = 512, 513
    d = tmp_path / "owl"
    save_hf_checkpoint(c.to_dict(), {k: v.contiguous() for k, v in sd.items() if "position_ids" not in k}, d)
    (d / "vocab.json").write_text(json.dumps(vocab))
    (d / "merges.txt").write_text("#version: 0.2\n")
    eng = InferenceEngine("cpu")
    pic = (torch.rand(48, 64, 3, generator=torch.Generator().manual_seed(2)) * 255).to(torch.uint8)
    res = eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="detect", images=[pic], texts=["a cat", "a dog"], score_threshold=0.0))
    dets = res.detections[0]
    assert dets and {x["label"] for x in dets} <= {"a cat", "a dog"} and all(0 <= x["score"] <= 1 for x in dets)
    assert dets == sorted(dets, key=lambda x: -x["score"])
    assert all(-70 <= x["box"][0] <= 70 and x["box"][2] >= x["box"][0] and x["box"][3] >= x["box"][1] for x in dets)
    none = eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="detect", images=[pic], texts=["a cat"], score_threshold=1.1))
    assert none.detections == [[]]
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="embed", images=[pic]))
    eng.close()


def test_mllama_vision_tower_and_cross_attention_match_transformers(tmp_path):
    """Llama 3.2 Vision end to end: tiled vision tower + projector + decoder with cross-attention
    layers against ``MllamaForConditionalGeneration`` on a two-tile image."""
    tr = pytest.importorskip("transformers")
    from transformers.models.mllama.configuration_mllama import MllamaConfig, MllamaTextConfig, MllamaVisionConfig
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from hartsyinference_b200.models.llm.transformer import ForwardBatch
    vc = MllamaVisionConfig(hidden_size=64, attention_heads=4, intermediate_size=128, num_hidden_layers=3, num_global_layers=2,
                            image_size=28, patch_size=14, max_num_tiles=4, intermediate_layers_indices=[0, 2], vision_output_dim=192)
    tc = MllamaTextConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                          num_key_value_heads=2, max_position_embeddings=256, cross_attention_layers=[1], pad_token_id=0,
                          rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    cfg = MllamaConfig(vision_config=vc, text_config=tc, image_token_index=319)
    cfg._attn_implementation = "eager"
    cfg.text_config._attn_implementation = "eager"
    cfg.vision_config._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.MllamaForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "embedding" not in n:
                p.mul_(2.0)
            if n.endswith("gate") or "cross_attn_attn_gate" in n or "cross_attn_mlp_gate" in n:
                p.fill_(0.6)                                   # the gates start at zero
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    hf = hf.to(torch.bfloat16).float()
    llm = load_llm(tmp_path / "m", "cpu")
    assert llm.vlm is not None and llm.config.cross_layers == (1,)
    g = torch.Generator().manual_seed(3)
    tiles = torch.zeros(4, 3, 28, 28)
    tiles[:2] = torch.randn(2, 3, 28, 28, generator=g)
    ids = [319] + torch.randint(0, 300, (14,), generator=g).tolist()          # the image token opens the prompt
    n = len(ids)
    ar_id = llm.vlm.tower.aspect_ratio_id(1, 2)
    with torch.no_grad():
        cam = torch.zeros(1, n, 1, 4)
        cam[..., :2] = 1
        ref = hf(input_ids=torch.tensor([ids]), pixel_values=tiles[None, None], aspect_ratio_ids=torch.tensor([[ar_id]]),
                 aspect_ratio_mask=torch.tensor([[[1, 1, 0, 0]]]), cross_attention_mask=cam).logits[0].float()
        plain = hf(input_ids=torch.tensor([ids])).logits[0].float()
    states = llm.vlm.encode_image(tiles, 1, 2)
    assert states.shape == (2 * 5, 128)
    m = llm.model
    m.alloc_kv(3, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32), block_table=torch.arange(3, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False, cu_q=torch.tensor([0, n], dtype=torch.int32),
                     max_q_len=n, max_kv_len=n, cross_states=states)
    mine = m.logits(m.forward_hidden(b)).float()
    cos = torch.nn.functional.cosine_similarity
    assert cos(ref.flatten(), plain.flatten(), dim=0) < 0.99
    assert cos(mine.flatten(), ref.flatten(), dim=0) > 0.99


def test_mllama_split_image_picks_the_tile_grid_by_aspect_ratio():
    from hartsyinference_b200.models.vlm.mllama import MllamaModel, MllamaVisionConfig, MllamaVisionTower
    cfg = MllamaVisionConfig(image_size=28, patch=14, max_tiles=4)
    glue = MllamaModel.__new__(MllamaModel)
    glue.tower = MllamaVisionTower.__new__(MllamaVisionTower)
    glue.tower.cfg = cfg
    wide = torch.rand(3, 40, 120)
    tiles, th, tw = glue.split_image(wide)
    assert (th, tw) == (1, 3) and tiles.shape == (4, 3, 28, 28)
    assert tiles[3].abs().sum() == 0 and tiles[2].abs().sum() > 0
    tall = torch.rand(3, 100, 50)
    assert glue.split_image(tall)[1:] == (2, 1)
    square = torch.rand(3, 64, 64)
    assert glue.split_image(square)[1:] == (2, 2)              # the largest grid of that shape
    assert glue.tower.aspect_ratio_id(2, 2) == 6


def _tiny_qwen_vl(tmp_path):
    tr = pytest.importorskip("transformers")
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "mrope_section": [4, 6, 6], "rope_theta": 10000.0}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, out_hidden_size=128, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1]),
        image_token_id=318, vision_start_token_id=317, vision_end_token_id=316, video_token_id=315)
    for c in (cfg, cfg.text_config, cfg.vision_config):
        c._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.Qwen2_5_VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    return hf.to(torch.bfloat16).float(), load_llm(tmp_path / "m", "cpu")


def test_qwen2_vl_matches_transformers(tmp_path):
    """The first Qwen-VL generation (LayerNorm tower, quick-GELU MLP, no windows) against
    ``Qwen2VLForConditionalGeneration``: vision features and an image prompt's greedy continuation."""
    tr = pytest.importorskip("transformers")
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLConfig
    from hartsyinference_b200.engine.llm_engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from hartsyinference_b200.models.vlm.qwen_vl import patchify
    cfg = Qwen2VLConfig(
        text_config=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "mrope_section": [4, 6, 6], "rope_theta": 10000.0}),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=14),
        image_token_id=318, vision_start_token_id=317, vision_end_token_id=316, video_token_id=315)
    for c in (cfg, cfg.text_config, cfg.vision_config):
        c._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.Qwen2VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    hf = hf.to(torch.bfloat16).float()
    llm = load_llm(tmp_path / "m", "cpu")
    assert llm.vlm.vision.cfg.legacy
    image = torch.rand(3, 56, 84, generator=torch.Generator().manual_seed(7))
    patches, gh, gw = patchify(image, llm.vlm.vision.cfg)
    with torch.no_grad():
        ref_feats = hf.model.visual(patches, grid_thw=torch.tensor([[1, gh, gw]])).pooler_output
    feats = llm.vlm.vision(patches, gh, gw)
    assert torch.nn.functional.cosine_similarity(feats.float().flatten(), ref_feats.flatten(), dim=0) > 0.99
    ids, embeds, mask, pos3, delta = llm.vlm.expand_prompt([5, 317, 318, 316, 20, 21, 22], [image])
    eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=96)
    rid = eng.add_request(ids, SamplingParams(greedy=True, max_tokens=5), prompt_embeds=embeds, embeds_mask=mask,
                          positions3=pos3, rope_delta=delta)
    eng.run_until_done()
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([[1, gh, gw]]),
                          max_new_tokens=5, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    assert eng.requests[rid].output[:len(ref)] == ref


def test_qwen2_5_vl_matches_transformers(tmp_path):
    """Windowed vision tower + merger + M-RoPE decoder against ``Qwen2_5_VLForConditionalGeneration``
    on a 6 x 8 patch image (3 x 4 merged tokens, two attention windows)."""
    from hartsyinference_b200.models.llm.transformer import ForwardBatch
    from hartsyinference_b200.models.vlm.qwen_vl import mrope_positions
    hf, llm = _tiny_qwen_vl(tmp_path)
    assert llm.vlm is not None and llm.config.mrope_section == (4, 6, 6)
    g = torch.Generator().manual_seed(4)
    gh, gw = 6, 8
    patches = torch.randn(gh * gw, 3 * 2 * 14 * 14, generator=g)
    feats = llm.vlm.vision(patches, gh, gw)
    with torch.no_grad():
        ref_feats = hf.model.visual(patches, grid_thw=torch.tensor([[1, gh, gw]])).pooler_output
    cos = torch.nn.functional.cosine_similarity
    assert feats.shape == (12, 128)
    assert cos(feats.float().flatten(), ref_feats.flatten(), dim=0) > 0.99
    ids = [5, 9, 317] + [318] * 12 + [316] + torch.randint(0, 300, (9,), generator=g).tolist()
    n = len(ids)
    pos3, delta = mrope_positions(ids, 318, [(3, 4)])
    assert pos3[:, 3:15].tolist() == [[3] * 12, [3, 3, 3, 3, 4, 4, 4, 4, 5, 5, 5, 5], [3, 4, 5, 6] * 3]
    assert pos3[:, 15].tolist() == [7, 7, 7] and delta == int(pos3.max()) + 1 - n
    with torch.no_grad():
        ref = hf(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([[1, gh, gw]]),
                 position_ids=pos3.long()[:, None, :]).logits[0].float()
    m = llm.model
    embeds = torch.zeros(n, 128, dtype=torch.bfloat16)
    mask = torch.tensor([t == 318 for t in ids])
    embeds[mask] = feats.to(torch.bfloat16)
    full = m.embed[torch.tensor(ids)].clone()
    full[mask] = embeds[mask]
    pages = (n + 15) // 16 + 1
    m.alloc_kv(pages, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32), block_table=torch.arange(pages, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False, cu_q=torch.tensor([0, n], dtype=torch.int32),
                     max_q_len=n, max_kv_len=n, embeds=full, positions3=pos3)
    mine = m.logits(m.forward_hidden(b)).float()
    assert cos(mine.flatten(), ref.flatten(), dim=0) > 0.99
    assert (mine.argmax(-1) == ref.argmax(-1)).float().mean() > 0.9


def test_qwen2_5_vl_engine_generation_follows_transformers(tmp_path):
    """An image prompt through the engine (three-axis prompt positions, shifted positions for the
    generated tokens, chunked prefill) continues like transformers' greedy generation; a text-only
    request batched with it is unaffected."""
    from hartsyinference_b200.engine.llm_engine import LLMEngine, SamplingParams
    hf, llm = _tiny_qwen_vl(tmp_path)
    g = torch.Generator().manual_seed(6)
    image = torch.rand(3, 84, 112, generator=g)
    prompt = [5, 9, 317, 318, 316] + torch.randint(0, 300, (6,), generator=g).tolist()
    ids, embeds, mask, pos3, delta = llm.vlm.expand_prompt(prompt, [image])
    assert len(ids) == len(prompt) - 1 + 12 and delta < 0
    other = torch.randint(0, 300, (11,), generator=g).tolist()
    sp = SamplingParams(greedy=True, max_tokens=6)

    def run(with_other, chunk):
        eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=4, prefill_chunk=chunk, max_model_len=96)
        rid = eng.add_request(ids, sp, prompt_embeds=embeds, embeds_mask=mask, positions3=pos3, rope_delta=delta)
        rid2 = eng.add_request(other, sp) if with_other else None
        eng.run_until_done()
        return eng.requests[rid].output, (eng.requests[rid2].output if with_other else None)

    out, out_other = run(True, 64)
    assert run(False, 8)[0] == out                              # chunked prefill slices the positions correctly
    eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=96)
    assert eng.generate([other], sp)[0] == out_other
    from hartsyinference_b200.models.vlm.qwen_vl import patchify
    patches, gh, gw = patchify(image, llm.vlm.vision.cfg)
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([[1, gh, gw]]),
                          max_new_tokens=6, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    assert out[:len(ref)] == ref


def test_qwen3_vl_matches_transformers(tmp_path):
    """Qwen3-VL: interpolated position table, deepstack taps added after the first decoder layers,
    interleaved three-axis rotary sections, against ``Qwen3VLForConditionalGeneration`` (vision
    features, deepstack features and the greedy continuation of an image prompt through the engine)."""
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, "Qwen3VLForConditionalGeneration"):
        pytest.skip("transformers has no Qwen3-VL")
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig
    from hartsyinference_b200.engine.llm_engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from hartsyinference_b200.models.vlm.qwen_vl import patchify
    cfg = Qwen3VLConfig(
        text_config=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "mrope_section": [6, 5, 5], "mrope_interleaved": True,
                                          "rope_theta": 10000.0}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, out_hidden_size=128, patch_size=16,
                           spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=16, deepstack_visual_indexes=[0, 2]),
        image_token_id=318, vision_start_token_id=317, vision_end_token_id=316, video_token_id=315)
    for c in (cfg, cfg.text_config, cfg.vision_config):
        c._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.Qwen3VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    hf = hf.to(torch.bfloat16).float()
    llm = load_llm(tmp_path / "m", "cpu")
    assert llm.config.mrope_interleaved and llm.config.qk_norm
    image = torch.rand(3, 64, 96, generator=torch.Generator().manual_seed(8))
    patches, gh, gw = patchify(image, llm.vlm.vision.cfg)
    assert (gh, gw) == (4, 6)
    with torch.no_grad():
        ref_out = hf.model.visual(patches, grid_thw=torch.tensor([[1, gh, gw]]))
    feats, taps = llm.vlm.vision(patches, gh, gw)
    cos = torch.nn.functional.cosine_similarity
    assert cos(feats.float().flatten(), ref_out.pooler_output.flatten(), dim=0) > 0.99
    assert len(taps) == 2
    for mine, ref in zip(taps, ref_out.deepstack_features):
        assert cos(mine.float().flatten(), ref.flatten(), dim=0) > 0.99
    ids, embeds, mask, pos3, delta = llm.vlm.expand_prompt([5, 317, 318, 316, 20, 21, 22], [image])
    assert llm.vlm.deepstack.shape == (2, len(ids), 128)
    outs = []
    for chunk in (64, 4):                                        # one-shot and chunked prefill
        eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=2, prefill_chunk=chunk, max_model_len=96)
        rid = eng.add_request(ids, SamplingParams(greedy=True, max_tokens=5), prompt_embeds=embeds, embeds_mask=mask,
                              positions3=pos3, rope_delta=delta, deepstack=llm.vlm.deepstack)
        eng.run_until_done()
        outs.append(eng.requests[rid].output)
    assert outs[0] == outs[1]
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([[1, gh, gw]]),
                          mm_token_type_ids=torch.tensor([[1 if t == 318 else 0 for t in ids]]),
                          max_new_tokens=5, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    assert outs[0][:len(ref)] == ref


def test_qwen_vl_and_mllama_checkpoints_through_text_service(tmp_path):
    """Image requests served end to end (prompt markers, vision tower, engine extras) for the two
    families that need more than replaced embeddings: Qwen2.5-VL and Llama 3.2 Vision."""
    import numpy as np
    tr = pytest.importorskip("transformers")
    from transformers.models.mllama.configuration_mllama import MllamaConfig, MllamaTextConfig, MllamaVisionConfig
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, TextRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    _tiny_qwen_vl(tmp_path / "q")
    vc = MllamaVisionConfig(hidden_size=64, attention_heads=4, intermediate_size=128, num_hidden_layers=2, num_global_layers=1,
                            image_size=28, patch_size=14, max_num_tiles=4, intermediate_layers_indices=[0], vision_output_dim=128)
    tc = MllamaTextConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                          num_key_value_heads=2, max_position_embeddings=256, cross_attention_layers=[1], pad_token_id=0,
                          rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    mcfg = MllamaConfig(vision_config=vc, text_config=tc, image_token_index=319)
    torch.manual_seed(0)
    hf = tr.MllamaForConditionalGeneration(mcfg)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("gate") or "cross_attn_attn_gate" in n or "cross_attn_mlp_gate" in n:
                p.fill_(0.8)
            elif p.ndim >= 2:
                p.mul_(3.0)
    save_hf_checkpoint(mcfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "mllama")
    img = (np.random.default_rng(0).random((56, 84, 3)) * 255).astype(np.uint8)
    other = (np.random.default_rng(1).random((56, 84, 3)) * 255).astype(np.uint8)
    eng = InferenceEngine("cpu")
    try:
        for d in (tmp_path / "q" / "m", tmp_path / "mllama"):
            spec = ModelSpec(str(d))
            text = eng.text.generate(spec, TextRequest(prompt="what is this?", max_tokens=4, greedy=True))
            a = eng.text.generate(spec, TextRequest(prompt="<image>what is this?", images=[img], max_tokens=4, greedy=True))
            again = eng.text.generate(spec, TextRequest(prompt="what is this?", images=[img], max_tokens=4, greedy=True))
            b = eng.text.generate(spec, TextRequest(prompt="<image>what is this?", images=[other], max_tokens=4, greedy=True))
            assert a.error is None and len(a.token_ids) == 4, a.error
            assert again.token_ids == a.token_ids                 # no placeholder: the image goes in front
            assert a.prompt_tokens > text.prompt_tokens
            logits_differ = a.token_ids != text.token_ids or a.token_ids != b.token_ids
            assert logits_differ, d
    finally:
        eng.text.release()
