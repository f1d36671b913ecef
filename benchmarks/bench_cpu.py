"""CPU decode benchmark: a Qwen2.5-0.5B-architecture decoder with random weights, batch 1, a prompt
of 128 uniformly drawn token ids and 128 greedy decode steps through the serving engine on the host
(PyTorch CPU path of every op), plus a logits check of the paged / chunked engine path against one
dense fp32 pass over the same tokens.

    python benchmarks/bench_cpu.py [--prompt 128] [--decode 128] [--threads N]

Prints one JSON line: decode tokens/s, prefill tokens/s, bytes of weights read per token, the
implied host bandwidth, and the parity figures.
"""
from __future__ import annotations

import argparse
import json
import time

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-native", action="store_true", help="skip the native host decoder (AVX-512 + thread team)")
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm.config import PRESETS
    from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
    cfg = PRESETS["qwen2.5-0.5b"]
    model = DecoderModel(cfg, "cpu")
    model.random_init(a.seed, std=0.02)
    g = torch.Generator().manual_seed(a.seed)
    prompt = torch.randint(0, cfg.vocab_size, (a.prompt,), generator=g).tolist()
    total = a.prompt + a.decode
    eng = LLMEngine(model, num_pages=(total + 15) // 16 + 2, page_size=16, max_batch=1, prefill_chunk=max(a.prompt, 16),
                    max_model_len=total + 16)
    rid = eng.add_request(prompt, SamplingParams(greedy=True, ignore_eos=True, max_tokens=a.decode))
    t0 = time.perf_counter()
    eng.step()                                   # prefill + first token
    t1 = time.perf_counter()
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    t2 = time.perf_counter()
    out = eng.requests[rid].output
    # parity: the engine's tokens against one dense causal pass over prompt + output (teacher forcing)
    seq = prompt + out[:-1]
    n = len(seq)
    model.alloc_kv((n + 15) // 16 + 1, 16)
    b = ForwardBatch(tokens=torch.tensor(seq, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32), block_table=torch.arange((n + 15) // 16 + 1, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False, cu_q=torch.tensor([0, n], dtype=torch.int32),
                     max_q_len=n, max_kv_len=n)
    logits = model.logits(model.forward_hidden(b)[a.prompt - 1:]).float()
    ref_tokens = logits.argmax(-1).tolist()
    agree = sum(int(x == y) for x, y in zip(ref_tokens, out)) / max(len(out), 1)
    top2 = logits.topk(2, -1).values
    weight_bytes = sum(lw.qkv.weight.numel() + lw.o.weight.numel() + lw.gate_up.weight.numel() + lw.down.weight.numel()
                       for lw in model.layers) * 4 + model.lm_head.weight.numel() * 4
    tok_s = steps / (t2 - t1) if t2 > t1 else 0.0
    native = None
    if not a.no_native:
        # the native host decoder on the same weights and prompt: greedy tokens must agree with the
        # engine's wherever the logits are not a near tie, and its last-step logits with the dense pass
        from hartsyinference_b200.models.llm.cpu_decoder import CpuDecoder
        dec = CpuDecoder(model, max_positions=total + 16, threads=a.threads)
        n0 = time.perf_counter()
        nxt = 0
        for t in prompt:
            nxt = dec.step(t)
        n1 = time.perf_counter()
        nat = [nxt]
        for _ in range(a.decode - 1):
            nat.append(dec.step(nat[-1]))
        n2 = time.perf_counter()
        nat_tok_s = (a.decode - 1) / (n2 - n1)
        # teacher-forced logits of the native path over the engine's own sequence
        dec.reset()
        lg = None
        forced = []
        for t in seq:
            g_tok, lg = dec.step(t, want_logits=True)
            forced.append(g_tok)
        forced = forced[a.prompt - 1:]
        cos = float(torch.nn.functional.cosine_similarity(lg, logits[-1, : cfg.vocab_size], dim=0))
        native = {"value": nat_tok_s, "unit": "tokens/s", "prefill_tok_s": a.prompt / (n1 - n0), "threads": dec.threads,
                  "simd_bits": dec.simd_bits, "implied_host_gbs": weight_bytes * nat_tok_s / 1e9,
                  "teacher_forced_token_agreement_with_engine": sum(int(x == y) for x, y in zip(forced, out)) / max(len(out), 1),
                  "last_logits_cosine_vs_dense_pass": cos}
    print(json.dumps({"metric": "decode tok/s (Qwen2.5-0.5B architecture, CPU fp32 math, batch 1)",
                      "value": native["value"] if native else tok_s, "unit": "tokens/s", "path": "native host decoder" if native else "op by op",
                      "op_by_op_tok_s": tok_s, "native": native,
                      "prompt": a.prompt, "decode": len(out), "prefill_tok_s": a.prompt / (t1 - t0), "threads": torch.get_num_threads(),
                      "weight_bytes_per_token": weight_bytes, "implied_host_gbs": weight_bytes * tok_s / 1e9,
                      "token_agreement_with_dense_pass": agree, "median_top1_top2_margin": float((top2[:, 0] - top2[:, 1]).median()),
                      "data": "synthetic: random-init weights N(0, 0.02) rounded to bf16, uniform-random prompt"}))


if __name__ == "__main__":
    main()
