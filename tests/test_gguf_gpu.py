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
