"""B200 runs of the breadth models against their CPU statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_clip_vision_tower_matches_cpu():
    from hartsyinference_b200.models.encoders.clip_vision import ClipVisionEncoder, tiny_clip_vision
    cfg = tiny_clip_vision()
    cpu = ClipVisionEncoder(cfg, "cpu", seed=4)
    gpu = ClipVisionEncoder(cfg, "cuda", seed=4)
    img = torch.randn(3, cfg.image_size, cfg.image_size, generator=torch.Generator().manual_seed(0))
    a = cpu.hidden_states(img, -2).float()
    b = gpu.hidden_states(img, -2).float().cpu()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.995


def test_whisper_matches_cpu():
    from hartsyinference_b200.models.audio import WhisperModel, tiny_whisper
    cfg = tiny_whisper()
    cpu, gpu = WhisperModel(cfg, "cpu", seed=2), WhisperModel(cfg, "cuda", seed=2)
    mel = torch.randn(cfg.n_mels, 2 * cfg.max_source, generator=torch.Generator().manual_seed(1))
    ea, eb = cpu.encode(mel), gpu.encode(mel)
    assert torch.nn.functional.cosine_similarity(ea.float().flatten(), eb.float().cpu().flatten(), dim=0) > 0.995
    toks = torch.tensor([3, 10, 20, 30], dtype=torch.int32)
    sa, sb = cpu.start(ea), gpu.start(eb)
    la = torch.cat([cpu.decode(sa, toks[:3]), cpu.decode(sa, toks[3:])])
    lb = torch.cat([gpu.decode(sb, toks[:3]), gpu.decode(sb, toks[3:])]).cpu()
    assert torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0) > 0.99


def test_llava_prefill_with_image_rows_on_device():
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.encoders.clip_vision import tiny_clip_vision
    from hartsyinference_b200.models.llm import config as C
    from hartsyinference_b200.models.llm.transformer import DecoderModel
    from hartsyinference_b200.models.vlm import LlavaModel
    outs = {}
    for dev in ("cpu", "cuda"):
        m = DecoderModel(C.tiny(), dev)
        m.random_init(3, std=0.05)
        vlm = LlavaModel(m, tiny_clip_vision(), m.cfg.vocab_size - 1, seed=5)
        img = torch.randn(3, 32, 32, generator=torch.Generator().manual_seed(1))
        ids, embeds, mask = vlm.expand_prompt([5, 9, m.cfg.vocab_size - 1, 11], [img])
        eng = LLMEngine(m, num_pages=64, page_size=16, max_batch=2, prefill_chunk=8, max_model_len=64)
        rid = eng.add_request(ids, SamplingParams(greedy=True, max_tokens=1), prompt_embeds=embeds, embeds_mask=mask)
        eng.run_until_done()
        outs[dev] = (embeds.float().cpu(), eng.requests[rid].output)
    assert torch.nn.functional.cosine_similarity(outs["cpu"][0].flatten(), outs["cuda"][0].flatten(), dim=0) > 0.99
    assert len(outs["cuda"][1]) == 1


_GPU_BASE = dict(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, max_position_embeddings=256)
_GPU_ARCHS = {
    "olmo2": ("Olmo2Config", {}),
    "gemma3_text": ("Gemma3TextConfig", dict(head_dim=64, sliding_window=8, query_pre_attn_scalar=64)),
    "glm4": ("Glm4Config", dict(head_dim=64, pad_token_id=0)),
    "starcoder2": ("Starcoder2Config", {}),
    "stablelm": ("StableLmConfig", dict(use_parallel_residual=True, use_qkv_bias=True)),
    "cohere": ("CohereConfig", {}),
    "nemotron": ("NemotronConfig", {}),
    "gpt_neox": ("GPTNeoXConfig", {}),
    "phi3": ("Phi3Config", dict(pad_token_id=0)),
    "olmoe": ("OlmoeConfig", dict(num_experts=4, num_experts_per_tok=2)),
    "bloom": ("BloomConfig", dict(n_layer=2, n_head=4)),
    "gpt_oss": ("GptOssConfig", dict(num_local_experts=4, num_experts_per_tok=2, head_dim=64, sliding_window=8,
                                     layer_types=["sliding_attention", "full_attention"])),
    "smollm3": ("SmolLM3Config", dict(pad_token_id=0, no_rope_layer_interval=2)),
    "exaone4": ("Exaone4Config", dict(head_dim=64)),
    "helium": ("HeliumConfig", dict(head_dim=64)),
    "hunyuan_v1_dense": ("HunYuanDenseV1Config", dict(head_dim=64)),
}


@pytest.mark.parametrize("name", sorted(_GPU_ARCHS))
def test_architecture_on_device_matches_cpu(name, tmp_path):
    """The block structures outside the fused decode path (LayerNorm with bias, parallel residual,
    post-block norms, q/k norm over all heads, partial rotary, non-gated FFNs) on the device kernels."""
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from hartsyinference_b200.models.llm.transformer import ForwardBatch
    cls, extra = _GPU_ARCHS[name]
    cfg = getattr(tr, cls)(**{**_GPU_BASE, **extra})
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg)
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
            else:
                p.add_(torch.randn_like(p) * 0.1)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, tmp_path / name)
    ids = torch.randint(0, 320, (37,), generator=torch.Generator().manual_seed(1)).tolist()
    outs = []
    for dev in ("cpu", "cuda"):
        m = load_llm(tmp_path / name, dev, fp8=False).model
        n = len(ids)
        pages = (n + 15) // 16 + 1
        m.alloc_kv(pages, 16)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        b = ForwardBatch(tokens=i32(ids), positions=i32(list(range(n))),
                         slot_mapping=torch.arange(n, dtype=torch.int64 if dev == "cuda" else torch.int32, device=dev),
                         block_table=i32(list(range(pages)))[None], kv_lens=i32([n]), is_decode=False,
                         cu_q=i32([0, n]), max_q_len=n, max_kv_len=n)
        outs.append(m.logits(m.forward_hidden(b)).float().cpu())
    cos = torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0)
    assert cos > 0.99, f"{name}: cos {cos:.4f}"


def test_mamba2_on_device_matches_cpu():
    from hartsyinference_b200.models.ssm import Mamba2Model, tiny_mamba2
    cfg = tiny_mamba2(n_groups=2)
    cpu, gpu = Mamba2Model(cfg, "cpu", seed=3), Mamba2Model(cfg, "cuda", seed=3)
    ids = torch.randint(0, 256, (19,), generator=torch.Generator().manual_seed(1))
    sa, sb = cpu.new_state(), gpu.new_state()
    la = torch.cat([cpu.logits(cpu.forward(ids[:12], sa)), cpu.logits(cpu.forward(ids[12:], sa))])
    lb = torch.cat([gpu.logits(gpu.forward(ids[:12], sb)), gpu.logits(gpu.forward(ids[12:], sb))]).cpu()
    assert torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0) > 0.99


def test_sd3_transformer_on_device_matches_cpu():
    from hartsyinference_b200.models.dit.sd3 import Sd3Transformer, tiny_sd3
    cfg = tiny_sd3(qk_norm=True)
    cpu, gpu = Sd3Transformer(cfg, "cpu", seed=2), Sd3Transformer(cfg, "cuda", seed=2)
    g = torch.Generator().manual_seed(1)
    lat = torch.randn(1, cfg.in_channels, 16, 16, generator=g)
    txt = torch.randn(1, 24, cfg.context_dim, generator=g)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g)
    sigma = torch.tensor([0.4])
    a = cpu.forward(lat, txt, sigma, pooled).float()
    b = gpu.forward(lat, txt, sigma, pooled).float().cpu()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.99


def test_chroma_on_device_matches_cpu():
    from hartsyinference_b200.models.dit import flux as F
    from hartsyinference_b200.models.dit.chroma import ChromaTransformer, tiny_chroma
    cfg = tiny_chroma(head_dim=64, num_heads=2, axes_dim=(16, 24, 24))
    cpu, gpu = ChromaTransformer(cfg, "cpu", seed=2), ChromaTransformer(cfg, "cuda", seed=2)
    g = torch.Generator().manual_seed(1)
    S_i, S_t = 64, 16
    img, txt = torch.randn(1, S_i, cfg.in_channels, generator=g), torch.randn(1, S_t, cfg.context_dim, generator=g)
    pooled = torch.zeros(1, cfg.pooled_dim)
    t = torch.tensor([0.5])
    outs = []
    for m, dev in ((cpu, "cpu"), (gpu, "cuda")):
        img_ids, txt_ids = F.flux_ids(8, 8, S_t, dev)
        outs.append(m.forward(img.to(dev), txt.to(dev), t.to(dev), pooled.to(dev), img_ids, txt_ids).float().cpu())
    assert torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0) > 0.99


def test_mllama_cross_attention_on_device_matches_cpu(tmp_path):
    """Llama 3.2 Vision decoder with vision states on the device kernels against the CPU path."""
    tr = pytest.importorskip("transformers")
    from transformers.models.mllama.configuration_mllama import MllamaTextConfig
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from hartsyinference_b200.models.llm.transformer import ForwardBatch
    cfg = MllamaTextConfig(**{**_GPU_BASE, "cross_attention_layers": [1], "num_hidden_layers": 3, "pad_token_id": 0,
                              "rope_parameters": {"rope_type": "default", "rope_theta": 10000.0}})
    torch.manual_seed(0)
    hf = tr.MllamaForCausalLM(cfg)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
            if n.endswith(("cross_attn_attn_gate", "cross_attn_mlp_gate")):
                p.fill_(0.7)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, tmp_path / "m")
    ids = torch.randint(0, 320, (29,), generator=torch.Generator().manual_seed(1)).tolist()
    states = torch.randn(24, 256, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    outs = []
    for dev in ("cpu", "cuda"):
        m = load_llm(tmp_path / "m", dev, fp8=False).model
        n = len(ids)
        pages = (n + 15) // 16 + 1
        m.alloc_kv(pages, 16)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        b = ForwardBatch(tokens=i32(ids), positions=i32(list(range(n))),
                         slot_mapping=torch.arange(n, dtype=torch.int64 if dev == "cuda" else torch.int32, device=dev),
                         block_table=i32(list(range(pages)))[None], kv_lens=i32([n]), is_decode=False,
                         cu_q=i32([0, n]), max_q_len=n, max_kv_len=n, cross_states=[states.to(dev)])
        outs.append(m.logits(m.forward_hidden(b)).float().cpu())
    cos = torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0)
    assert cos > 0.99, f"cos {cos:.4f}"


def test_qwen_vl_three_axis_rotary_on_device_matches_cpu(tmp_path):
    """Qwen2.5-VL: vision tower, merged-token embeddings and the three-section rotary embedding on
    the device against the CPU path, through the engine."""
    tr = pytest.importorskip("transformers")
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig
    from hartsyinference_b200.engine.llm_engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "mrope_section": [8, 12, 12], "rope_theta": 10000.0}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, out_hidden_size=256, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1]),
        image_token_id=318, vision_start_token_id=317, vision_end_token_id=316, video_token_id=315)
    torch.manual_seed(0)
    hf = tr.Qwen2_5_VLForConditionalGeneration(cfg)
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, tmp_path / "m")
    image = torch.rand(3, 84, 112, generator=torch.Generator().manual_seed(6))
    prompt = [5, 9, 317, 318, 316, 40, 41, 42, 43]
    outs = {}
    for dev in ("cpu", "cuda"):
        llm = load_llm(tmp_path / "m", dev, fp8=False)
        ids, embeds, mask, pos3, delta = llm.vlm.expand_prompt(prompt, [image])
        eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=96)
        rid = eng.add_request(ids, SamplingParams(greedy=True, max_tokens=4), prompt_embeds=embeds, embeds_mask=mask,
                              positions3=pos3, rope_delta=delta)
        eng.run_until_done()
        outs[dev] = (embeds.float().cpu(), eng.requests[rid].output)
    assert torch.nn.functional.cosine_similarity(outs["cpu"][0].flatten(), outs["cuda"][0].flatten(), dim=0) > 0.99
    assert len(outs["cuda"][1]) == 4 and outs["cuda"][1][0] == outs["cpu"][1][0]


def test_qwen35_hybrid_on_device_matches_cpu():
    """Qwen3.5 hybrid (gated DeltaNet + gated attention) on the device GEMM / GLU kernels against the CPU path."""
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, "Qwen3_5ForCausalLM"):
        pytest.skip("transformers has no Qwen3.5")
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from hartsyinference_b200.models.ssm import Qwen35Model, qwen35_from_hf
    hf_cfg = Qwen3_5TextConfig(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=64, linear_conv_kernel_dim=4, linear_key_head_dim=32,
                               linear_value_head_dim=32, linear_num_key_heads=4, linear_num_value_heads=8,
                               max_position_embeddings=256, pad_token_id=0)
    torch.manual_seed(0)
    hf = tr.Qwen3_5ForCausalLM(hf_cfg)
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = qwen35_from_hf(hf_cfg.to_dict())
    ids = torch.randint(0, 320, (24,), generator=torch.Generator().manual_seed(1))
    outs = []
    for dev in ("cpu", "cuda"):
        m = Qwen35Model(cfg, dev, get=lambda n: sd.get(n))
        st = m.new_state()
        m.forward(ids[:16], st)
        outs.append(m.logits(m.forward(ids[16:], st)).float().cpu())
    cos = torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0)
    assert cos > 0.99, f"cos {cos:.4f}"
