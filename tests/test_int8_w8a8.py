"""W8A8 linear (int8 operands on tcgen05 kind::i8, per-row / per-channel scales in the epilogue) and
the ConvRot codec. Oracle: fp32 ``x @ W^T`` of the unquantised operands (tolerance of 8-bit
quantisation), and exact integer arithmetic of the quantised operands."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.assets import int8_convrot as C


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


def test_rotation_is_orthogonal_symmetric_and_matches_the_matrix():
    for g in (4, 16, 64, 256):
        h = C.hadamard(g)
        assert float((h @ h - torch.eye(g)).abs().max()) < 1e-5
        assert float((h - h.t()).abs().max()) < 1e-6
        x = torch.randn(3, 2 * g)
        want = torch.cat([x[:, :g] @ h, x[:, g:] @ h], 1)
        assert float((C.rotate(x, g) - want).abs().max()) < 1e-4
    assert not C.is_valid_group(8) and not C.is_valid_group(2) and C.is_valid_group(1024)
    with pytest.raises(ValueError):
        C.rotate(torch.randn(2, 24), 16)


def test_weight_round_trip_and_cpu_linear():
    torch.manual_seed(0)
    w = torch.randn(96, 256) * 0.1
    for g in (0, 16, 256):
        q, s = C.quantize_weight(w, g)
        assert q.dtype == torch.int8 and s.shape == (96,)
        assert _rel(C.dequant_to_bf16(q, s, g), w) < 0.02
        x = torch.randn(5, 256).to(torch.bfloat16)
        lw = ops.Int8Weight.from_dense(w, torch.randn(96), g)
        y = ops.linear(x, lw)
        assert _rel(y, x.float() @ w.t() + lw.bias.float()) < 0.03, g


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(64, 512, 1024), (300, 768, 512), (1, 256, 256), (1000, 1536, 2048)])
@pytest.mark.parametrize("group", [0, 16, 256])
def test_device_int8_linear(m, n, k, group):
    torch.manual_seed(1)
    x = (torch.randn(m, k, device="cuda") * 0.7).to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda") * 0.05
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    lw = ops.Int8Weight.from_dense(w, bias, group)
    got = ops.linear(x, lw, act="gelu_tanh")
    # exact statement of what the kernels compute: same quantised operands, integer dot products
    qx, sx = C.quantize_activation(x.cpu(), group)
    acc = qx.double() @ lw.weight.cpu().double().t()
    want = torch.nn.functional.gelu((acc * sx.double()[:, None] * lw.row_scale.cpu().double()[None, :]).float() + bias.cpu().float(),
                                    approximate="tanh")
    assert _rel(got.cpu(), want) < 8e-3, _rel(got.cpu(), want)
    # and close to the unquantised product
    full = torch.nn.functional.gelu(x.float() @ w.t() + bias.float(), approximate="tanh")
    assert _rel(got, full) < 0.05


@pytest.mark.gpu
def test_device_activation_quantiser_matches_statement():
    torch.manual_seed(2)
    x = (torch.randn(37, 1024, device="cuda") * 2).to(torch.bfloat16)
    sm = (0.5 + torch.rand(1024, device="cuda")).float()
    for group in (0, 64):
        q, s = ops.quant_int8_act(x, group, sm)
        qr, sr = C.quantize_activation(x.cpu(), group, sm.cpu())
        assert float((s.cpu() - sr).abs().max() / sr.abs().max()) < 1e-5
        assert int((q.cpu().int() - qr.int()).abs().max()) <= 1       # rounding of values that sit on .5
