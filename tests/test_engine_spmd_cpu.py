"""Multi-process engine on CPU ranks (gloo): tensor-parallel text generation and CFG-parallel image
generation through ``InferenceEngine`` / the CLI must reproduce the single-process results."""
import hashlib
import os
import subprocess
import sys

import pytest

from hartsyinference_b200.engine.inference_engine import InferenceEngine
from hartsyinference_b200.engine.requests import EngineOptions, ImageRequest, Modality, ModelSpec, TextRequest
from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
from tests.test_llm_loader_cpu import _synthetic

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    d = tmp_path_factory.mktemp("spmd")
    cfg, t = _synthetic(seed=5)
    save_hf_checkpoint(cfg, t, d / "toy")
    return str(d / "toy")


def _torchrun(args, port, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port)] + args
    e = dict(os.environ, CUDA_VISIBLE_DEVICES="", **(env or {}))
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=e)


def test_tensor_parallel_text_through_the_engine(ckpt):
    res = _torchrun([os.path.join(ROOT, "tests", "mp_engine_spmd_cpu_worker.py"), ckpt, "text"], 29561)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = next(l for l in res.stdout.splitlines() if l.startswith("SPMD_TEXT"))
    eng = InferenceEngine("cpu", EngineOptions(max_batch=8, max_model_len=256, kv_pool_bytes_budget=8 << 20), ranks=None)
    spec = ModelSpec(ckpt, Modality.TEXT, local_path=ckpt)
    a = eng.text.generate(spec, TextRequest(prompt="hello world", greedy=True, max_tokens=8))
    assert str(a.token_ids) in line, (a.token_ids, line)
    eng.close()


def test_cfg_parallel_image_through_the_engine():
    res = _torchrun([os.path.join(ROOT, "tests", "mp_engine_spmd_cpu_worker.py"), "-", "image"], 29562)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = next(l for l in res.stdout.splitlines() if l.startswith("SPMD_IMAGE"))
    eng = InferenceEngine("cpu", ranks=None)
    r = eng.images.generate(ModelSpec("synthetic:flux-tiny", Modality.IMAGE),
                            ImageRequest(prompt="a cat", negative_prompt="blurry", width=64, height=64, steps=2, cfg_scale=3.0, seed=3))
    assert hashlib.sha256(r.rgb).hexdigest() in line
    eng.close()


def test_cli_relaunches_itself_for_tp2(ckpt):
    """``cli text --tp 2`` on one process starts two ranks and prints the generation once."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT="29563", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-m", "hartsyinference_b200.cli", "text", ckpt, "hello", "--raw", "--greedy",
                          "--max-tokens", "6", "--device", "cpu", "--tp", "2"], capture_output=True, text=True, timeout=600,
                         cwd=ROOT, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "tokens, ttft" in res.stderr and res.stderr.count("tokens, ttft") == 1
