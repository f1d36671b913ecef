"""Dense tcgen05 attention (head dim 128, bidirectional) against the fp32 statement."""
import math

import pytest
import torch

from hartsyinference_b200 import config, ops
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.fixture
def tc_attention():
    config.set_override("tc_attention", True)
    yield
    config.set_override("tc_attention", None)


@pytest.mark.parametrize("tq,tk,heads", [(256, 256, 2), (128, 512, 1), (300, 1000, 3), (1024, 4608, 2), (77, 333, 4)])
def test_tc_attention_matches_fp32(tq, tk, heads, tc_attention):
    torch.manual_seed(tq + tk)
    q = torch.randn(tq, heads, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(tk, heads, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(tk, heads, 128, device="cuda").to(torch.bfloat16)
    out = ops.attention(q, k, v)
    N.check_status()
    ref = R.attention(q.cpu(), k.cpu(), v.cpu(), False, 1.0 / math.sqrt(128), 0.0, 0)
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 2e-2, err
    # and against the mma.sync kernel
    config.set_override("tc_attention", False)
    base = ops.attention(q, k, v)
    config.set_override("tc_attention", True)
    assert (out.float() - base.float()).abs().max().item() < 2e-2


def test_tc_attention_large_scores_and_determinism(tc_attention):
    torch.manual_seed(0)
    q = (torch.randn(384, 2, 128, device="cuda") * 3).to(torch.bfloat16)
    k = (torch.randn(640, 2, 128, device="cuda") * 3).to(torch.bfloat16)
    v = torch.randn(640, 2, 128, device="cuda").to(torch.bfloat16)
    a = ops.attention(q, k, v)
    b = ops.attention(q, k, v)
    assert torch.equal(a, b) and torch.isfinite(a.float()).all()
    ref = R.attention(q.cpu(), k.cpu(), v.cpu(), False, 1.0 / math.sqrt(128), 0.0, 0)
    assert (a.float().cpu() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("tq,tk,heads", [(256, 256, 2), (128, 512, 1), (300, 1000, 3), (1024, 4608, 2), (77, 333, 4), (513, 2049, 1)])
def test_fa_attention_matches_fp32(tq, tk, heads, int8):
    """Two-query-tile kernel with S / P / O in TMEM, bf16 and int8 (SageAttention) score modes,
    against fp32 attention. The int8 tolerance is the one of per-row int8 quantisation of Q and K."""
    config.set_override("fa_attention", True)
    try:
        torch.manual_seed(tq * 7 + tk)
        q = torch.randn(tq, heads, 128, device="cuda").to(torch.bfloat16)
        k = (torch.randn(tk, heads, 128, device="cuda") + 0.5).to(torch.bfloat16)      # non-zero mean: the smoothing matters
        v = torch.randn(tk, heads, 128, device="cuda").to(torch.bfloat16)
        out = ops.attention(q, k, v, int8=int8)
        N.check_status()
        ref = R.attention(q.cpu(), k.cpu(), v.cpu(), False, 1.0 / math.sqrt(128), 0.0, 0)
        err = (out.float().cpu() - ref).abs().max().item()
        rel = ((out.float().cpu() - ref).norm() / ref.norm()).item()
        assert err < (6e-2 if int8 else 2e-2) and rel < (3e-2 if int8 else 1e-2), (err, rel)
    finally:
        config.set_override("fa_attention", None)


def test_fa_attention_rescale_path_and_determinism():
    """Scores that keep growing along the keys force the lazy running-maximum update (O rescaled in
    TMEM) many times; results must stay finite, exact to tolerance and bit-identical across runs."""
    config.set_override("fa_attention", True)
    try:
        torch.manual_seed(0)
        tq, tk = 384, 1536
        q = (torch.randn(tq, 2, 128, device="cuda") * 2).to(torch.bfloat16)
        k = (torch.randn(tk, 2, 128, device="cuda") * torch.linspace(0.2, 4.0, tk, device="cuda")[:, None, None]).to(torch.bfloat16)
        v = torch.randn(tk, 2, 128, device="cuda").to(torch.bfloat16)
        for int8 in (False, True):
            a = ops.attention(q, k, v, int8=int8)
            b = ops.attention(q, k, v, int8=int8)
            N.check_status()
            assert torch.equal(a, b) and torch.isfinite(a.float()).all()
            ref = R.attention(q.cpu(), k.cpu(), v.cpu(), False, 1.0 / math.sqrt(128), 0.0, 0)
            if int8:
                # very peaked softmax rows amplify the int8 rounding of the scores: judge the bulk
                rel = ((a.float().cpu() - ref).norm() / ref.norm()).item()
                assert rel < 0.2, rel
            else:
                assert (a.float().cpu() - ref).abs().max().item() < 3e-2
    finally:
        config.set_override("fa_attention", None)
