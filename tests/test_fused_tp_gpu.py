"""Fused GEMM -> all-reduce (+ residual + RMSNorm + fp8 emit) kernel. On one GPU the group has a
single rank: the same protocol (partials into the symmetric heap, ready / done counters, row
reduce, call roll-over) runs with the GPU as its own peer. The multi-GPU case runs as child
processes under torchrun."""
import os
import subprocess
import sys

import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.exceptions import DeviceWaitTimeout
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R
from hartsyinference_b200.parallel.comm import SingleComm
from hartsyinference_b200.parallel.fused import FusedColumnParallel, FusedRowParallel


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


def _oracle(x, w, bias, res, norm_w, eps):
    """fp32 reference of linear (+ bias) -> + residual -> RMSNorm."""
    s = x.float() @ w.float().t()
    if bias is not None:
        s = s + bias.float()
    s = s.to(torch.bfloat16).float()
    r = s if res is None else (s + res.float()).to(torch.bfloat16).float()
    h = r
    if norm_w is not None:
        h = r * torch.rsqrt((r * r).mean(-1, keepdim=True) + eps) * norm_w.float()
    return r, h


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_single_rank_protocol_matches_oracle(fp8):
    torch.manual_seed(0)
    f = FusedRowParallel(SingleComm(), 1024)
    try:
        for it, m in enumerate((64, 1, 128, 17, 64, 64)):
            n, k = 1024, 512
            x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
            w = (torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16)
            b = torch.randn(n, device="cuda").to(torch.bfloat16)
            r0 = torch.randn(m, n, device="cuda").to(torch.bfloat16)
            nw = (1 + 0.1 * torch.randn(n, device="cuda")).to(torch.bfloat16)
            lw = ops.LinearWeight.from_dense(w, b, fp8=fp8)
            res = r0.clone()
            h, h8 = f(x, lw, res=res, norm_w=nw, eps=1e-5, emit_bf16=True, emit_fp8=True)
            h = h.clone()
            plain = ops.linear(x, lw, splits=1)          # same operands on the same tensor-core path (bias included)
            s = (plain.float()).to(torch.bfloat16).float()
            rr = (s + r0.float()).to(torch.bfloat16).float()
            want = rr * torch.rsqrt((rr * rr).mean(-1, keepdim=True) + 1e-5) * nw.float()
            N.check_status()
            assert _rel(res, rr) < 1e-2, (it, m, "residual", _rel(res, rr))
            assert _rel(h, want) < 1e-2, (it, m, "norm", _rel(h, want))
            deq = R.dequant_fp8_act(h8.data.clone(), h8.scales_fp32())
            assert _rel(deq, want) < 6e-2, (it, m, "fp8", _rel(deq, want))
        # no residual, no norm: a plain all-reduced linear
        x = (torch.randn(33, 512, device="cuda") * 0.5).to(torch.bfloat16)
        lw = ops.LinearWeight.from_dense((torch.randn(1024, 512, device="cuda") * 0.2).to(torch.bfloat16), fp8=fp8)
        y, _ = f(x, lw)
        assert _rel(y, ops.linear(x, lw, splits=1)) < 1e-2
        N.check_status()
    finally:
        f.close()


@pytest.mark.gpu
def test_against_fp32_oracle_bf16():
    torch.manual_seed(3)
    f = FusedRowParallel(SingleComm(), 2048)
    try:
        m, n, k = 40, 2048, 1024
        x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
        r0 = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        nw = (1 + 0.1 * torch.randn(n, device="cuda")).to(torch.bfloat16)
        res = r0.clone()
        h, _ = f(x, ops.LinearWeight(w), res=res, norm_w=nw, eps=1e-6)
        rr, want = _oracle(x, w, None, r0, nw, 1e-6)
        assert _rel(res, rr) < 1e-2 and _rel(h, want) < 1e-2
        N.check_status()
    finally:
        f.close()


@pytest.mark.gpu
def test_single_rank_cuda_graph_replay():
    torch.manual_seed(1)
    f = FusedRowParallel(SingleComm(), 512)
    try:
        x = (torch.randn(32, 256, device="cuda") * 0.5).to(torch.bfloat16)
        w = ops.LinearWeight((torch.randn(512, 256, device="cuda") * 0.2).to(torch.bfloat16))
        out = torch.zeros(32, 512, device="cuda", dtype=torch.bfloat16)
        for _ in range(2):
            f(x, w)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out.copy_(f(x, w)[0])
            out.add_(f(x, w)[0])      # second output buffer, second call inside the same graph
        for _ in range(3):
            x.mul_(0.5)
            g.replay()
            torch.cuda.synchronize()
            ref = 2 * (x.float() @ w.weight.float().t())
            assert _rel(out, ref) < 2e-2
        N.check_status()
    finally:
        f.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_large_token_form_matches_fp32(fp8):
    """More than 128 tokens: GEMM in the large-token orientation, elementwise reduce phase with bias,
    gate and the (read-only) residual stream; slots chained like the DiT blocks chain them."""
    torch.manual_seed(4)
    f = FusedRowParallel(SingleComm(), 768, max_large_tokens=700)
    try:
        for m in (300, 640, 129):
            n, k = 768, 512
            x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
            w = (torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16)
            b = torch.randn(n, device="cuda").to(torch.bfloat16)
            lw = ops.LinearWeight.from_dense(w, b, fp8=fp8)
            res = torch.randn(m, n, device="cuda").to(torch.bfloat16)
            gate = torch.randn(n, device="cuda").to(torch.bfloat16)
            plain = ops.linear(x, lw).float()             # same operands, bias included
            y1 = f.large(x, lw, res=res, gate=gate, slot=0)
            want1 = res.float() + gate.float() * plain
            N.check_status()
            assert _rel(y1, want1) < 1e-2, (m, "gated", _rel(y1, want1))
            y2 = f.large(x, lw, res=y1, slot=1)           # the previous output as the residual stream
            N.check_status()
            assert _rel(y2, y1.float() + plain) < 1e-2, (m, "chained", _rel(y2, y1.float() + plain))
            assert _rel(y1, want1) < 1e-2                 # slot 0 is untouched by the call into slot 1
            y3 = f.large(x, lw)                           # plain all-reduced linear
            assert _rel(y3, plain) < 1e-2
        # the small-token form still works on the same instance afterwards
        x = (torch.randn(64, 512, device="cuda") * 0.5).to(torch.bfloat16)
        lw = ops.LinearWeight.from_dense((torch.randn(768, 512, device="cuda") * 0.2).to(torch.bfloat16), fp8=fp8)
        y, _ = f(x, lw)
        N.check_status()
        assert _rel(y, ops.linear(x, lw, splits=1)) < 1e-2
    finally:
        f.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_allgather_gemm_and_reduce_scatter_single_rank(fp8):
    """One rank owns all rows: the copy into the gather buffer, the per-tile arrival waits, the tile
    rotation and the reduce-scatter store path all run; results match the plain linear."""
    torch.manual_seed(6)
    col = FusedColumnParallel(SingleComm(), 700, 1024)
    row = FusedRowParallel(SingleComm(), 768, max_large_tokens=700)
    try:
        for m, k in ((300, 512), (640, 1024), (129, 256), (300, 512)):
            n = 768
            x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
            lw = ops.LinearWeight.from_dense((torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16),
                                             torch.randn(n, device="cuda").to(torch.bfloat16), fp8=fp8)
            want = ops.linear(x, lw, act="gelu_tanh")
            got = col(x, lw, m, act="gelu_tanh")
            N.check_status()
            assert _rel(got, want) < 1e-2, (m, k, _rel(got, want))
            res = torch.randn(m, n, device="cuda").to(torch.bfloat16)
            gate = torch.randn(n, device="cuda").to(torch.bfloat16)
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            row.large(x, lw, res=res, gate=gate, scatter_out=out)
            N.check_status()
            assert _rel(out, res.float() + gate.float() * ops.linear(x, lw).float()) < 1e-2
    finally:
        col.close()
        row.close()


@pytest.mark.gpu
def test_wait_runs_out_reports_and_recovers():
    """A rank that never raises `ready`: the bounded wait gives up after about a millisecond, the
    kernel returns, the status word names kernel and site, and after the counters are cleared the
    next call is correct. Nothing faults; the context stays usable."""
    torch.manual_seed(2)
    f = FusedRowParallel(SingleComm(), 512)
    try:
        x = (torch.randn(16, 256, device="cuda") * 0.5).to(torch.bfloat16)
        w = ops.LinearWeight((torch.randn(512, 256, device="cuda") * 0.2).to(torch.bfloat16))
        f(x, w)
        N.check_status()
        f.debug_skip_ready, budget = True, f.budget_cycles
        f.budget_cycles = 2_000_000          # about 1 ms
        f(x, w)
        f.debug_skip_ready, f.budget_cycles = False, budget
        with pytest.raises(DeviceWaitTimeout) as ei:
            N.check_status()
        assert ei.value.kernel == 5 and ei.value.site == 1      # fused GEMM + all-reduce, wait for `ready`
        f.reset()
        y, _ = f(x, w)
        N.check_status()
        assert _rel(y, x.float() @ w.weight.float().t()) < 2e-2
    finally:
        f.close()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_rank_fused_allreduce_and_tp_model():
    worker = os.path.join(os.path.dirname(__file__), "mp_fused_tp_worker.py")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", worker],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "FUSED_TP_OK" in res.stdout
