"""Device sampler (csrc/kernels/sampling.cu) against the fp32 statement of the chain
(ops.reference.sampling_keep_mask): every drawn token lies in the kept set, the empirical
distribution over many draws follows the renormalised probabilities, greedy rows are the argmax,
and a (seed, counter) pair always gives the same token."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import reference as R


def _params(rows, t, k, p, mp, seed0=0, counter0=0, dev="cuda"):
    return (torch.full((rows,), t, dtype=torch.float32, device=dev), torch.full((rows,), k, dtype=torch.int32, device=dev),
            torch.full((rows,), p, dtype=torch.float32, device=dev), torch.full((rows,), mp, dtype=torch.float32, device=dev),
            torch.arange(seed0, seed0 + rows, dtype=torch.int64, device=dev), torch.full((rows,), counter0, dtype=torch.int64, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("t,k,p,mp", [(0.8, 50, 0.9, 0.0), (1.0, 0, 0.95, 0.0), (0.7, 20, 0.0, 0.0), (1.2, 0, 0.0, 0.05),
                                      (1.0, 0, 0.0, 0.0), (0.9, 40, 0.8, 0.02)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_draws_stay_inside_the_kept_set(t, k, p, mp, dtype):
    torch.manual_seed(0)
    vocab, rows = 32000, 16
    base = (torch.randn(rows, vocab, device="cuda") * 3.0).to(dtype)
    keep = torch.stack([R.sampling_keep_mask(base[r].float(), t, k, p, mp) for r in range(rows)])
    for counter in range(8):
        tok = ops.sample_tokens(base, *_params(rows, t, k, p, mp, seed0=100, counter0=counter))
        assert bool(keep[torch.arange(rows), tok.long()].all()), (counter, tok.tolist())
    a = ops.sample_tokens(base, *_params(rows, t, k, p, mp, seed0=7, counter0=3))
    b = ops.sample_tokens(base, *_params(rows, t, k, p, mp, seed0=7, counter0=3))
    assert torch.equal(a, b)


@pytest.mark.gpu
def test_empirical_distribution_follows_the_probabilities():
    torch.manual_seed(1)
    vocab, rows = 64, 4096
    row = torch.randn(vocab, device="cuda") * 1.5
    logits = row[None].expand(rows, vocab).contiguous()
    t, k, p, mp = 0.9, 12, 0.92, 0.0
    keep = R.sampling_keep_mask(row, t, k, p, mp)
    want = torch.softmax((row / t).masked_fill(~keep, float("-inf")), -1)
    tok = ops.sample_tokens(logits, *_params(rows, t, k, p, mp, seed0=1000))
    freq = torch.bincount(tok.long(), minlength=vocab).float() / rows
    assert bool(keep[tok.long()].all())
    assert float((freq - want).abs().max()) < 0.03, (freq - want).abs().max()


@pytest.mark.gpu
def test_greedy_rows_and_mixed_batch():
    torch.manual_seed(2)
    vocab, rows = 151936, 6
    logits = torch.randn(rows, vocab, device="cuda")
    logits[2, 777] = logits[2, 99] = 50.0            # a tie: the lower id wins
    temp, k, p, mp, seed, ctr = _params(rows, 0.0, 0, 0.0, 0.0)
    temp[4:] = 0.8
    k[4:] = 1                                          # top-1 sampling is the argmax too
    tok = ops.sample_tokens(logits, temp, k, p, mp, seed, ctr)
    want = logits.argmax(-1)
    want[2] = 99
    assert tok.tolist() == want.tolist()


def test_cpu_statement_runs():
    torch.manual_seed(3)
    logits = torch.randn(3, 100)
    tok = ops.sample_tokens(logits, *_params(3, 0.8, 10, 0.9, 0.0, dev="cpu"))
    for r in range(3):
        assert bool(R.sampling_keep_mask(logits[r], 0.8, 10, 0.9, 0.0)[int(tok[r])])
