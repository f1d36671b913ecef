"""Worker of the regroup test: three CPU ranks (gloo) run a tensor-parallel toy decoder; after the
first step rank 2 leaves (between steps, nothing in flight, exit code 0). The others notice it
through the heartbeats before their next collective, agree on the survivors, form a two-rank
group, re-shard the model for tp=2 and produce the same logits as the single-rank model.
Arguments: port."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.parallel.elastic import ElasticGroup


def weights(cfg):
    g = torch.Generator().manual_seed(3)
    full = {}
    mk = lambda n, *s: full.__setitem__(n, (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16))
    H, F, V = cfg.hidden_size, cfg.ffn_size, cfg.vocab_size
    mk("model.embed_tokens.weight", V, H); mk("lm_head.weight", V, H)
    full["model.norm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        mk(p + "self_attn.q_proj.weight", cfg.q_size, H); mk(p + "self_attn.k_proj.weight", cfg.kv_size, H)
        mk(p + "self_attn.v_proj.weight", cfg.kv_size, H); mk(p + "self_attn.o_proj.weight", H, cfg.q_size)
        mk(p + "mlp.gate_proj.weight", F, H); mk(p + "mlp.up_proj.weight", F, H); mk(p + "mlp.down_proj.weight", H, F)
        full[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        full[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    return full


def logits(cfg, full, comm):
    t = 12
    toks = torch.arange(t, dtype=torch.int32) % cfg.vocab_size
    m = DecoderModel(cfg, "cpu", comm=comm)
    m.load_state_dict(full.get)
    m.alloc_kv(4, 16)
    b = ForwardBatch(tokens=toks, positions=torch.arange(t, dtype=torch.int32), slot_mapping=torch.arange(t, dtype=torch.int64),
                     block_table=torch.arange(4, dtype=torch.int32)[None], kv_lens=torch.tensor([t], dtype=torch.int32),
                     is_decode=False, cu_q=torch.tensor([0, t], dtype=torch.int32), max_q_len=t, max_kv_len=t)
    return m.full_logits(m.forward_hidden(b)).float()


def main():
    port = int(sys.argv[1])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    # 6 heads / 6 kv heads, ffn 384, vocab 384: divisible by 3 and by 2
    cfg = C.tiny("llama-3-70b", vocab_size=384, hidden_size=192, num_layers=2, num_heads=6, num_kv_heads=6, head_dim=32, ffn_size=384)
    full = weights(cfg)
    eg = ElasticGroup(rank, world, "127.0.0.1", port, backend="gloo", timeout_s=20.0)
    step1 = logits(cfg, full, eg.comm)               # tp = 3
    eg.beat()
    if rank == 2:
        eg.comm.barrier()                            # the step is over everywhere
        eg.leave()
        eg.close()
        return 0
    eg.comm.barrier()
    # -------- between steps: who is still there?
    deadline = time.time() + 15
    while not eg.dead(timeout_s=1.0) and time.time() < deadline:
        time.sleep(0.1)
        eg.beat()
    assert eg.dead(timeout_s=1.0) == [2], eg.dead(timeout_s=1.0)
    survivors = eg.agree_on_survivors(timeout_s=1.0)
    assert survivors == [0, 1], survivors
    comm = eg.regroup(survivors)                     # tp = 2
    assert comm.world == 2 and comm.rank == rank
    step2 = logits(cfg, full, comm)
    if rank == 0:
        from hartsyinference_b200.parallel.comm import SingleComm
        ref = logits(cfg, full, SingleComm())
        c1 = torch.nn.functional.cosine_similarity(step1, ref, dim=-1).min().item()
        c2 = torch.nn.functional.cosine_similarity(step2, ref, dim=-1).min().item()
        assert c1 > 0.999 and c2 > 0.999, (c1, c2)
        print("ELASTIC_OK", round(c1, 5), round(c2, 5), flush=True)
    comm.barrier()
    eg.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
