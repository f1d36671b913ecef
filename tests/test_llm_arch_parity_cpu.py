"""Every decoder architecture the config factory claims, checked against transformers: a tiny
random model of that family is saved as a checkpoint directory, loaded through ``load_llm`` and its
prefill logits are compared with the Hugging Face forward of the same weights."""
import pytest
import torch

from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
from hartsyinference_b200.models.llm.transformer import ForwardBatch

tr = pytest.importorskip("transformers")

_BASE = dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=256)

ARCHS = {
    "llama": ("LlamaConfig", dict(rope_theta=10000.0)),
    "llama3_rope": ("LlamaConfig", dict(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                       "high_freq_factor": 4.0, "original_max_position_embeddings": 64})),
    "mistral": ("MistralConfig", dict(sliding_window=None)),
    "qwen2": ("Qwen2Config", dict()),
    "qwen3": ("Qwen3Config", dict(head_dim=32)),
    "gemma": ("GemmaConfig", dict(head_dim=32)),
    "gemma2": ("Gemma2Config", dict(head_dim=32, sliding_window=8, query_pre_attn_scalar=32)),
    "gemma3_text": ("Gemma3TextConfig", dict(head_dim=32, sliding_window=8, query_pre_attn_scalar=32)),
    "granite": ("GraniteConfig", dict(residual_multiplier=0.5, embedding_multiplier=3.0, logits_scaling=2.0,
                                      attention_multiplier=0.2)),
    "olmo2": ("Olmo2Config", dict()),
    "mixtral": ("MixtralConfig", dict(num_local_experts=4, num_experts_per_tok=2)),
    "qwen2_moe": ("Qwen2MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                         shared_expert_intermediate_size=128, decoder_sparse_step=1, mlp_only_layers=[])),
    "qwen3_moe": ("Qwen3MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, head_dim=32,
                                         decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)),
    "olmoe": ("OlmoeConfig", dict(num_experts=4, num_experts_per_tok=2)),
}


def _logits(llm, ids):
    m = llm.model
    n = len(ids)
    m.alloc_kv((n + 15) // 16 + 1, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32),
                     block_table=torch.arange((n + 15) // 16 + 1, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False,
                     cu_q=torch.tensor([0, n], dtype=torch.int32), max_q_len=n, max_kv_len=n)
    return m.logits(m.forward_hidden(b)).float()


@pytest.mark.parametrize("name", sorted(ARCHS))
def test_arch_matches_transformers(name, tmp_path):
    cls, extra = ARCHS[name]
    if not hasattr(tr, cls):
        pytest.skip(f"transformers has no {cls}")
    cfg = getattr(tr, cls)(**{**_BASE, **extra})
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():            # default init is tiny; widen so that every branch matters
            if p.ndim >= 2:
                p.mul_(3.0)
            elif "norm" in "".join(n for n, q in hf.named_parameters() if q is p):
                p.add_(torch.randn_like(p) * 0.1)
    d = tmp_path / name
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, d)
    hf = hf.to(torch.bfloat16).float()       # the same rounded weights on both sides
    llm = load_llm(d, "cpu")
    ids = torch.randint(0, 320, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        ref = hf(torch.tensor([ids])).logits[0].float()
    mine = _logits(llm, ids)
    cos = torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0)
    assert cos > 0.995, f"{name}: cos {cos:.4f}"
    agree = (mine.argmax(-1) == ref.argmax(-1)).float().mean()
    assert agree >= 0.85, f"{name}: argmax agreement {agree:.2f}"
