"""In-tree build of the native libraries.

Three shared objects are produced under ``hartsyinference_b200/lib``:

* ``libb200_kernels.so``  every ``csrc/kernels/*.cu`` compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); plain C ABI, no PyTorch headers, loaded with
  ctypes and called with raw device pointers and the current CUDA stream.
* ``libb200_runtime.so``  host-side C++ runtime (``csrc/runtime/*.cpp``): safetensors / GGUF
  readers, GGUF block codecs, paged-KV block allocator, continuous-batching scheduler core,
  BPE tokenizer. No CUDA dependency, so it builds and is tested on CPU-only machines.
* ``libb200infer.so``     the public C ABI (``csrc/cabi/*.c``) that hosts the Python engine.

The reference ships PTX that the driver JIT-compiles at load time
(src/HartsyInference.Cuda/CudaModule.cs, Kernels/README.md:39); here everything is compiled
ahead of time and nothing is JIT-ed.

Usage: ``python -m hartsyinference_b200.build [--force] [--verbose]``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import json
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "550,177",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, flush=True)


def _load_stamp() -> dict:
    f = LIB / "build_stamp.json"
    if f.exists():
        try:
            return json.loads(f.read_text())
        except Exception:
            return {}
    return {}


def _save_stamp(stamp: dict) -> None:
    (LIB / "build_stamp.json").write_text(json.dumps(stamp, indent=1))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link ``libb200_kernels.so``."""
    out = LIB / "libb200_kernels.so"
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h"))
    stamp = _load_stamp()
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_digest = _digest(hdrs, " ".join(NVCC_FLAGS))
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        d = _digest([s], hdr_digest)
        if force or not o.exists() or stamp.get(f"obj:{s.name}") != d:
            jobs.append((s, o, d))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {
                ex.submit(_run, [nvcc, *NVCC_FLAGS, "-I", str(CSRC / "kernels"), "-c", str(s), "-o", str(o)], verbose): (s, d)
                for s, o, d in jobs
            }
            for f in cf.as_completed(futs):
                f.result()
                s, d = futs[f]
                stamp[f"obj:{s.name}"] = d
    link_digest = hashlib.sha256("".join(stamp.get(f"obj:{s.name}", "") for s in srcs).encode()).hexdigest()
    if force or jobs or not out.exists() or stamp.get("kernels") != link_digest:
        _run([nvcc, "-shared", "-o", str(out), *[str(o) for o in objs], "-gencode",
              "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose)
        stamp["kernels"] = link_digest
    _save_stamp(stamp)
    return out


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    """Build the host-side C++ runtime (no CUDA)."""
    out = LIB / "libb200_runtime.so"
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    hdrs = sorted((CSRC / "runtime").glob("*.h")) + sorted((CSRC / "runtime").glob("*.hpp"))
    if not srcs:
        return out
    stamp = _load_stamp()
    d = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    if force or not out.exists() or stamp.get("runtime") != d:
        LIB.mkdir(parents=True, exist_ok=True)
        cxx = os.environ.get("CXX", "g++")
        _run([cxx, *CXX_FLAGS, "-shared", "-o", str(out), *[str(s) for s in srcs], "-I", str(CSRC / "runtime")], verbose)
        stamp["runtime"] = d
        _save_stamp(stamp)
    return out


def build_cabi(force: bool = False, verbose: bool = False) -> Path:
    """Build the public C ABI library, which embeds CPython to host the engine."""
    out = LIB / "libb200infer.so"
    srcs = sorted((CSRC / "cabi").glob("*.c")) + sorted((CSRC / "cabi").glob("*.cpp"))
    hdrs = sorted((CSRC / "cabi").glob("*.h"))
    if not srcs:
        return out
    stamp = _load_stamp()
    d = _digest(srcs + hdrs, "cabi")
    if force or not out.exists() or stamp.get("cabi") != d:
        inc = sysconfig.get_paths()["include"]
        libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
        ver = sysconfig.get_config_var("LDVERSION") or "3"
        cc = os.environ.get("CC", "gcc")
        _run([cc, "-O2", "-fPIC", "-shared", "-o", str(out), *[str(s) for s in srcs], "-I", inc,
              "-I", str(CSRC / "cabi"), f"-L{libdir}", f"-lpython{ver}", "-ldl", "-pthread"], verbose)
        stamp["cabi"] = d
        _save_stamp(stamp)
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    LIB.mkdir(parents=True, exist_ok=True)
    return {
        "kernels": build_kernels(force, verbose),
        "runtime": build_runtime(force, verbose),
        "cabi": build_cabi(force, verbose),
    }


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    libs = build_all(args.force, args.verbose)
    for k, v in libs.items():
        print(f"{k}: {v} ({'ok' if v.exists() else 'no sources'})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
