"""Worker of the SPMD engine test: every rank builds the same InferenceEngine; rank 0 generates
text through the public API with the model sharded over both ranks (tp=2) and an image with the
two guidance branches on the two ranks (cfg-parallel); the other rank follows. Results must equal
the single-process engine's. Launched under torchrun with CPU (gloo) ranks."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hartsyinference_b200.engine.inference_engine import InferenceEngine
from hartsyinference_b200.engine.requests import EngineOptions, ImageRequest, Modality, ModelSpec, TextRequest
from hartsyinference_b200.parallel.config import ParallelConfig


def main():
    ckpt, mode = sys.argv[1], sys.argv[2]
    placement = ParallelConfig(tp=2) if mode == "text" else ParallelConfig(cfg=2)
    eng = InferenceEngine("cpu", EngineOptions(placement=placement, max_batch=8, max_model_len=256,
                                               kv_pool_bytes_budget=8 << 20))
    if not eng.is_front:
        eng.follow()
        return
    assert eng.ready() == {"ranks": 2, "healthy": [True, True]}
    if mode == "text":
        spec = ModelSpec(ckpt, Modality.TEXT, local_path=ckpt)
        a = eng.text.generate(spec, TextRequest(prompt="hello world", greedy=True, max_tokens=8))
        b = eng.text.generate(spec, TextRequest(prompt="hello world", temperature=0.8, seed=7, max_tokens=8))
        c = eng.text.generate(spec, TextRequest(prompt="hello world", temperature=0.8, max_tokens=6))     # seed drawn by rank 0
        print("SPMD_TEXT", a.token_ids, b.token_ids, len(c.token_ids), flush=True)
    else:
        spec = ModelSpec("synthetic:flux-tiny", Modality.IMAGE)
        r = eng.images.generate(spec, ImageRequest(prompt="a cat", negative_prompt="blurry", width=64, height=64, steps=2,
                                                   cfg_scale=3.0, seed=3))
        import hashlib
        print("SPMD_IMAGE", hashlib.sha256(r.rgb).hexdigest(), r.width, r.height, flush=True)
    eng.close()


if __name__ == "__main__":
    main()
