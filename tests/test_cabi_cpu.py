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
