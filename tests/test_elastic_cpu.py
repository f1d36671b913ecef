"""Failure detection and regrouping on the host (CPU ranks, gloo): a rank that leaves between steps
is noticed through its heartbeat, the survivors form a smaller group and re-shard the model."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rank_leaves_between_steps_and_the_group_regroups_at_lower_degree():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    procs = []
    for r in range(3):
        e = dict(env, RANK=str(r), WORLD_SIZE="3")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_elastic_cpu_worker.py"), "29571"],
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT, env=e))
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (so, se) in zip(procs, outs):
        assert p.returncode == 0, so[-2000:] + se[-4000:]
    assert "ELASTIC_OK" in outs[0][0]
