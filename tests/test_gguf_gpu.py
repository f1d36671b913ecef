"""GGUF block formats consumed on the device: dequantisation kernels and the integer-dot GEMV
against the host codec (fp32)."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.assets import gguf as G

pytestmark = pytest.mark.gpu


def _make(ggml_type, n, k, seed=0):
    torch.manual_seed(seed)
    w = torch.randn(n, k) * 0.05
    raw = G.quantize(w, ggml_type)                      # uint8 blocks (host codec)
    ref = G.dequantize(raw, ggml_type, n * k).reshape(n, k)
    gw = ops.GgufWeight.from_raw(torch.as_tensor(raw).cuda(), ggml_type, n, k)
    return gw, ref


@pytest.mark.parametrize("ggml_type", [ops.core.GGML_Q8_0, ops.core.GGML_Q4_K])
def test_device_dequant_matches_host_codec(ggml_type):
    gw, ref = _make(ggml_type, 96, 1024)
    got = gw.dequantize().float().cpu()
    assert (got - ref).abs().max() <= ref.abs().max() * 2 ** -8      # bf16 rounding only


@pytest.mark.parametrize("ggml_type", [ops.core.GGML_Q8_0, ops.core.GGML_Q4_K])
@pytest.mark.parametrize("m", [1, 2, 5, 8, 16, 40])
def test_gguf_linear_matches_dequantised_product(ggml_type, m):
    n, k = 320, 2048
    gw, ref = _make(ggml_type, n, k, seed=m)
    gw.bias = (torch.randn(n) * 0.1).to(torch.bfloat16).cuda()
    x = (torch.randn(m, k) * 0.5).to(torch.bfloat16).cuda()
    y = ops.gguf_linear(x, gw).float().cpu()
    want = x.float().cpu() @ ref.t() + gw.bias.float().cpu()
    err = (y - want).abs().max() / want.abs().max()
    assert err < 0.02, err                                             # int8 activations: < 1 % typical


def test_resident_gguf_model_generates_like_the_dequantised_one(tmp_path):
    from hartsyinference_b200 import config
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm.loader import load_llm
    from tests.test_llm_loader_cpu import _synthetic, _to_gguf
    cfg, t = _synthetic(5, qkv_bias=False, heads=4, kvh=2, d=64)      # head dim the device kernels support
    _to_gguf(cfg, t, tmp_path / "q.gguf", quant=G.GGML_TYPES["Q8_0"])
    dense = load_llm(tmp_path / "q.gguf", "cuda", fp8=False)
    config.set_override("gguf_resident", True)
    try:
        res = load_llm(tmp_path / "q.gguf", "cuda", fp8=False)
    finally:
        config.set_override("gguf_resident", None)
    assert isinstance(res.model.layers[0].qkv, ops.GgufWeight)
    p = SamplingParams(greedy=True, max_tokens=8, ignore_eos=True)
    prompts = [[3, 9, 27, 81, 5], [7, 7, 7]]
    outs = []
    for m in (dense.model, res.model):
        e = LLMEngine(m, num_pages=32, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=128)
        outs.append(e.generate(prompts, p))
    # int8 activations in the GEMV: agreement on the first tokens, not bit equality
    assert sum(a[:2] == b[:2] for a, b in zip(*outs)) >= 1
    assert all(len(o) == 8 for o in outs[1])
