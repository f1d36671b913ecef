"""Fused GEMM -> all-reduce kernel. On one GPU the group has a single rank: the same protocol
(push to the owner's staging, flag, owner reduce, push result, completion count, epoch roll-over)
runs with the GPU as its own peer. The multi-GPU case runs as child processes under torchrun."""
import os
import subprocess
import sys

import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.parallel.comm import SingleComm
from hartsyinference_b200.parallel.fused import FusedRowParallel


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_single_rank_protocol_matches_plain_gemm(fp8):
    torch.manual_seed(0)
    f = FusedRowParallel(SingleComm(), 1024)
    try:
        for it, m in enumerate((64, 1, 128, 17, 64, 64)):
            n, k = 1024, 512
            x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
            w = (torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16)
            b = torch.randn(n, device="cuda").to(torch.bfloat16)
            r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
            lw = ops.LinearWeight.from_dense(w, b, fp8=fp8)
            y = f(x, lw, residual=r).clone()
            ref = ops.linear(x, lw, residual=r, splits=1)
            N.check_status()
            assert _rel(y, ref) < 1e-2, (it, m, _rel(y, ref))
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
            out.copy_(f(x, w))
            out.add_(f(x, w))      # second output buffer, second call inside the same graph
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
@pytest.mark.multigpu
def test_two_rank_fused_allreduce_and_tp_model():
    worker = os.path.join(os.path.dirname(__file__), "mp_fused_tp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", worker],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "FUSED_TP_OK" in res.stdout
