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
