"""Engine on a B200: fused kernels + CUDA-graph decode must reproduce the CPU oracle's tokens."""
import pytest
import torch

from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel
from hartsyinference_b200.ops import _native as N

pytestmark = pytest.mark.gpu


def _pair(fp8: bool, seed: int, **kw):
    cfg = C.tiny("llama-3-70b", vocab_size=1024, hidden_size=512, num_layers=3, num_heads=8, num_kv_heads=2,
                 head_dim=128, ffn_size=1024, **kw)
    g = DecoderModel(cfg, "cuda", fp8=fp8)
    g.random_init(seed, std=0.05)
    return cfg, g


def _cpu_copy(g: DecoderModel) -> DecoderModel:
    c = DecoderModel(g.cfg, "cpu", fp8=g.fp8)
    from hartsyinference_b200.ops import LinearWeight
    mv = lambda t: None if t is None else t.cpu()
    c.embed, c.final_norm = g.embed.cpu(), g.final_norm.cpu()
    c.lm_head = LinearWeight(mv(g.lm_head.weight), mv(g.lm_head.scale), mv(g.lm_head.bias))
    from hartsyinference_b200.models.llm.transformer import LayerWeights
    for lw in g.layers:
        c.layers.append(LayerWeights(
            in_norm=lw.in_norm.cpu(), post_norm=lw.post_norm.cpu(),
            qkv=LinearWeight(mv(lw.qkv.weight), mv(lw.qkv.scale), mv(lw.qkv.bias)),
            o=LinearWeight(mv(lw.o.weight), mv(lw.o.scale), mv(lw.o.bias)),
            gate_up=LinearWeight(mv(lw.gate_up.weight), mv(lw.gate_up.scale), mv(lw.gate_up.bias)),
            down=LinearWeight(mv(lw.down.weight), mv(lw.down.scale), mv(lw.down.bias)),
            q_norm=mv(lw.q_norm), k_norm=mv(lw.k_norm)))
    return c


@pytest.mark.parametrize("fp8", [False, True])
def test_gpu_prefill_logits_match_cpu_oracle(fp8):
    cfg, g = _pair(fp8, 1)
    c = _cpu_copy(g)
    from hartsyinference_b200.models.llm.transformer import ForwardBatch
    t = 70
    torch.manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (t,), dtype=torch.int32)

    def run(m, dev):
        m.alloc_kv(8, 16)
        b = ForwardBatch(tokens=toks.to(dev), positions=torch.arange(t, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(t, dtype=torch.int64, device=dev),
                         block_table=torch.arange(8, dtype=torch.int32, device=dev)[None],
                         kv_lens=torch.tensor([t], dtype=torch.int32, device=dev), is_decode=False,
                         cu_q=torch.tensor([0, t], dtype=torch.int32, device=dev), max_q_len=t, max_kv_len=t)
        return m.full_logits(m.forward_hidden(b)).float().cpu()

    lg, lc = run(g, "cuda"), run(c, "cpu")
    N.check_status()
    cos = torch.nn.functional.cosine_similarity(lg, lc, dim=-1)
    assert cos.min().item() > (0.99 if fp8 else 0.999), cos.min().item()


@pytest.mark.parametrize("fp8,graphs", [(False, True), (True, True), (True, False)])
def test_gpu_engine_generation_matches_cpu(fp8, graphs):
    cfg, g = _pair(fp8, 2)
    c = _cpu_copy(g)
    torch.manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (40, 7, 90)]
    p = SamplingParams(greedy=True, ignore_eos=True, max_tokens=12)
    eg = LLMEngine(g, num_pages=64, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=256,
                   use_cuda_graphs=graphs)
    ec = LLMEngine(c, num_pages=64, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=256)
    og, oc = eg.generate(prompts, p), ec.generate(prompts, p)
    N.check_status()
    # greedy decisions can legitimately differ at near-ties of a random toy model (and every later
    # token then differs too): require the first token of most prompts and one longer common prefix
    assert sum(a[:1] == b[:1] for a, b in zip(og, oc)) >= 2, (og, oc)
    assert sum(a[:4] == b[:4] for a, b in zip(og, oc)) >= 1, (og, oc)
    assert all(len(o) == 12 for o in og)
    if graphs:
        assert len(eg._graphs) >= 1 and not eg._graphs_disabled


def test_graph_and_eager_decode_agree_exactly():
    cfg, g = _pair(True, 3)
    torch.manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (33, 64, 5, 17)]
    p = SamplingParams(greedy=True, ignore_eos=True, max_tokens=10)
    outs = []
    for graphs in (True, False):
        e = LLMEngine(g, num_pages=64, page_size=16, max_batch=4, prefill_chunk=128, max_model_len=256,
                      use_cuda_graphs=graphs)
        outs.append(e.generate(prompts, p))
    assert outs[0] == outs[1]


def test_smoke_entry():
    import __graft_entry__ as ge
    ge.smoke()
