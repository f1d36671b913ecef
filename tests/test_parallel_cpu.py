"""Multi-rank logic on CPU ranks (gloo, world size 2): TP, Ulysses SP, CFG-parallel, comm ops."""
import os
import subprocess
import sys

import torch

from hartsyinference_b200.parallel.config import ParallelConfig


def _torchrun(script, port, n=2, timeout=300):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), script],
                          capture_output=True, text=True, timeout=timeout, env=env)


def test_two_cpu_ranks_match_single_rank():
    res = _torchrun(os.path.join(os.path.dirname(__file__), "mp_parallel_cpu_worker.py"), 29551)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "PARALLEL_CPU_OK" in res.stdout


def test_parallel_config_roundtrip():
    for s in ("single", "tp8", "sp4+cfg2", "tp2+pp2", "ep8+dp8"):
        assert ParallelConfig.parse(s).describe() == s
    assert ParallelConfig(tp=2, cfg=2).world_size == 4 and ParallelConfig().is_single
    assert ParallelConfig(sp=4, cfg=2).cache_key != ParallelConfig(sp=8).cache_key
