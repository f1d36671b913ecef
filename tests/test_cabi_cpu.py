"""The C ABI, driven from a stand-alone C program (embedded interpreter) and in-process via ctypes."""
import ctypes as C
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

import pytest

from hartsyinference_b200 import build
from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
from tests.test_llm_loader_cpu import _synthetic

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    d = tmp_path_factory.mktemp("cabi")
    cfg, t = _synthetic(seed=9)
    save_hf_checkpoint(cfg, t, d / "toy")
    return d


def test_c_program_round_trip(ckpt):
    lib = build.build_cabi()
    inc = ROOT / "hartsyinference_b200" / "csrc" / "cabi"
    exe = ckpt / "harness"
    subprocess.run(["gcc", "-O1", "-o", str(exe), str(ROOT / "tests" / "cabi_harness.c"), f"-I{inc}", f"-L{lib.parent}",
                    "-lb200infer", f"-Wl,-rpath,{lib.parent}"], check=True)
    site = sysconfig.get_paths()["purelib"]
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{site}", OMP_NUM_THREADS="2")
    res = subprocess.run([str(exe), str(ckpt / "toy")], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, (res.returncode, res.stdout[-2000:], res.stderr[-3000:])
    assert "CABI_OK" in res.stdout


def test_in_process_via_ctypes(ckpt):
    lib = C.CDLL(str(build.build_cabi()))
    lib.b200_last_error.restype = C.c_char_p
    eng = C.c_void_p()
    assert lib.b200_engine_create(b"cpu", b'{"max_model_len": 128, "max_batch": 2, "kv_pool_bytes_budget": 4194304}', C.byref(eng)) == 0
    out = C.c_char_p()
    spec = ('{"requested": "%s"}' % (ckpt / "toy")).encode()
    rc = lib.b200_text_generate(eng, spec, b'{"prompt": "a", "max_tokens": 3, "greedy": true}', C.byref(out))
    assert rc == 0, lib.b200_last_error()
    assert b"completion_tokens" in out.value
    assert lib.b200_engine_set_backend(eng, b"vulkan") == 4          # UnsupportedBackendError code
    assert b"Vulkan" in lib.b200_last_error()
    lib.b200_engine_destroy(eng)


def test_new_modalities_via_ctypes(ckpt, tmp_path):
    """Embeddings, upscaling and speech through the C entry points (buffers in, buffers out)."""
    import json
    import numpy as np
    import torch
    from hartsyinference_b200.assets.safetensors import save_file
    from tests.test_audio_cpu import _vits_hf
    from tests.test_restore_cpu import _Net
    lib = C.CDLL(str(build.build_cabi()))
    lib.b200_last_error.restype = C.c_char_p
    eng = C.c_void_p()
    assert lib.b200_engine_create(b"cpu", b'{"max_model_len": 128, "max_batch": 2, "kv_pool_bytes_budget": 4194304}', C.byref(eng)) == 0
    spec = ('{"requested": "%s"}' % (ckpt / "toy")).encode()
    out, count, dim = C.POINTER(C.c_float)(), C.c_int(), C.c_int()
    rc = lib.b200_embed_text(eng, spec, b'["hello", "world!"]', C.byref(out), C.byref(count), C.byref(dim))
    assert rc == 0, lib.b200_last_error()
    emb = np.ctypeslib.as_array(out, shape=(count.value, dim.value)).copy()
    lib.b200_free(out)
    assert emb.shape == (2, 128) and np.allclose(np.linalg.norm(emb, axis=1), 1.0, atol=1e-3)

    torch.manual_seed(2)
    save_file({k: v.detach().contiguous() for k, v in _Net(8, 1, 4, 4).state_dict().items()}, tmp_path / "esrgan.safetensors")
    rgb = bytes(np.random.default_rng(0).integers(0, 255, 12 * 10 * 3, dtype=np.uint8))
    up, w, h = C.POINTER(C.c_uint8)(), C.c_int(), C.c_int()
    uspec = ('{"requested": "%s"}' % (tmp_path / "esrgan.safetensors")).encode()
    rc = lib.b200_upscale(eng, uspec, b'{"tile": 0}', rgb, 12, 10, C.byref(up), C.byref(w), C.byref(h))
    assert rc == 0, lib.b200_last_error()
    assert (w.value, h.value) == (48, 40)
    lib.b200_free(up)

    c, hf = _vits_hf()
    d = tmp_path / "voice"
    save_hf_checkpoint(c.to_dict(), {k: v.detach().float().contiguous() for k, v in hf.state_dict().items()
                                     if not k.startswith("posterior_encoder")}, d)
    (d / "vocab.json").write_text(json.dumps({"<pad>": 0, **{ch: i + 1 for i, ch in enumerate("abcdefghijklmnopqrstuvwxyz ")}}))
    pcm, n, rate = C.POINTER(C.c_float)(), C.c_longlong(), C.c_int()
    rc = lib.b200_speak(eng, ('{"requested": "%s"}' % d).encode(), b'{"text": "hello there"}', C.byref(pcm), C.byref(n), C.byref(rate))
    assert rc == 0, lib.b200_last_error()
    wave = np.ctypeslib.as_array(pcm, shape=(n.value,)).copy()
    lib.b200_free(pcm)
    assert rate.value == 16000 and n.value > 0 and np.abs(wave).max() <= 1.0
    assert lib.b200_speak(eng, b'{"requested": "/no/such/voice"}', b'{"text": "x"}', C.byref(pcm), C.byref(n), C.byref(rate)) != 0
    assert lib.b200_music(eng, b'{"requested": "/no/such/model"}', b'{"prompt": "x", "seconds": 0.1}', C.byref(pcm), C.byref(n), C.byref(rate)) != 0
    assert b"No such file" in lib.b200_last_error() or len(lib.b200_last_error()) > 0
    lib.b200_engine_destroy(eng)
