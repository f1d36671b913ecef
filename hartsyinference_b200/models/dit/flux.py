"""Flux-class rectified-flow image DiT (double-stream + single-stream blocks) over the fused ops.

Architecture (Flux.1-Dev: 19 double + 38 single blocks, hidden 3072, 24 heads x 128, MLP ratio 4,
RoPE axes [16, 56, 56], theta 10000; src/HartsyInference.Diffusion/Models/Denoisers/FluxConfig.cs:
37-58). Block op order follows the reference's ``FluxDoubleStreamBlock`` (6 linears :230-242, QK
RMSNorm :247-257, joint attention :295, projections :322, gated residuals :325-349) and
``FluxSingleStreamBlock`` (fused qkv+mlp linear :139-153, attention :188, GELU :200, output linear
:223), with the elementwise work folded into kernels: LayerNorm + AdaLN modulation (+ fp8 emit) is
one launch, qkv split + QK-norm + RoPE is one launch, GELU / gate / residual live in GEMM epilogues.

Tensor parallelism: heads and MLP columns are split across the group (column-parallel qkv / mlp-in,
row-parallel proj / mlp-out), two all-reduces per stream per double block and one per single block.
The reference splits Flux by blocks across two GPUs instead (``ForwardSharded``,
FluxTransformer.cs:288-404); that pipeline split is available through ``block_range``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import config, log, ops
from ...ops import LinearWeight
from ...parallel.comm import Comm, SingleComm
from .common import WeightFactory, modulation, rope_tables, silu, timestep_embedding


@dataclass(frozen=True)
class FluxConfig:
    in_channels: int = 64
    hidden_size: int = 3072
    num_heads: int = 24
    head_dim: int = 128
    num_double_blocks: int = 19
    num_single_blocks: int = 38
    mlp_ratio: float = 4.0
    context_dim: int = 4096
    pooled_dim: int = 768
    axes_dim: tuple = (16, 56, 56)
    theta: float = 10000.0
    guidance_embed: bool = True
    out_channels: int = 0            # 0 = in_channels; the Fill / Canny / Depth variants read more channels than they predict

    @property
    def latent_channels(self) -> int:
        return self.out_channels or self.in_channels

    @property
    def mlp_dim(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)


FLUX_DEV = FluxConfig()
# Structural-conditioning variants (FLUX.1 Canny / Depth): the control image's latents ride along
# the noisy latents channel-wise; FLUX.1 Fill adds the 8 x 8-folded mask (64 + 64 + 256 channels).
FLUX_CONTROL = FluxConfig(in_channels=128, out_channels=64)
FLUX_FILL = FluxConfig(in_channels=384, out_channels=64)


def tiny_flux(**over) -> FluxConfig:
    kw = dict(in_channels=16, hidden_size=128, num_heads=4, head_dim=32, num_double_blocks=2, num_single_blocks=2,
              context_dim=64, pooled_dim=32, axes_dim=(8, 12, 12))
    kw.update(over)
    return FluxConfig(**kw)


@dataclass
class _StreamWeights:
    mod: LinearWeight            # 6 * H modulation
    qkv: LinearWeight
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    proj: LinearWeight
    mlp_in: LinearWeight
    mlp_out: LinearWeight


@dataclass
class _SingleWeights:
    mod: LinearWeight            # 3 * H modulation
    qkv_mlp: LinearWeight        # [3 * Hl * D + mlp_local, H]
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    out: LinearWeight            # [H, Hl * D + mlp_local]


class FluxTransformer:
    # Variants whose AdaLN vectors do not come from per-block linears of the time / text embedding
    # (Chroma) set this to False: those linears and the embedders are then not built.
    HAS_MODULATION_LINEARS = True

    def __init__(self, cfg: FluxConfig = FLUX_DEV, device="cpu", comm: Optional[Comm] = None, fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0,
                 block_range: Optional[tuple[int, int]] = None, build_head: bool = True, stream_blocks: bool = False):
        """``stream_blocks``: every transformer block moves to pinned host memory as soon as it is built
        (device peak: embedders + one block) and the forward pass streams them through two device slots
        (engine/block_streaming.py); chosen by the engine's VRAM planner when the weights do not fit."""
        self.cfg = cfg
        self.has_head = build_head
        self.device = torch.device(device)
        self.comm = comm or SingleComm()
        self.tp, self.tp_rank = self.comm.world, self.comm.rank
        assert cfg.num_heads % self.tp == 0 and cfg.mlp_dim % self.tp == 0
        self.hl = cfg.num_heads // self.tp
        self.mlp_l = cfg.mlp_dim // self.tp
        H, D = cfg.hidden_size, cfg.head_dim
        f = WeightFactory(self.device, fp8, self.tp_rank, self.tp, get, seed)
        self.fp8 = fp8 and self.device.type == "cuda"
        total_blocks = cfg.num_double_blocks + cfg.num_single_blocks
        self.block_range = block_range or (0, total_blocks)
        first, last = self.block_range[0] == 0, self.block_range[1] == total_blocks
        self.x_embedder = f.linear("x_embedder", H, cfg.in_channels, allow_fp8=False) if first else None
        self.context_embedder = f.linear("context_embedder", H, cfg.context_dim) if first else None
        mods = self.HAS_MODULATION_LINEARS
        lin_mod = (lambda name, n: f.linear(name, n * H, H)) if mods else (lambda name, n: None)
        if mods:
            self.t_in = f.linear("time_text_embed.timestep_embedder.linear_1", H, 256, allow_fp8=False)
            self.t_out = f.linear("time_text_embed.timestep_embedder.linear_2", H, H)
        if mods and cfg.guidance_embed:
            self.g_in = f.linear("time_text_embed.guidance_embedder.linear_1", H, 256, allow_fp8=False)
            self.g_out = f.linear("time_text_embed.guidance_embedder.linear_2", H, H)
        if mods:
            self.p_in = f.linear("time_text_embed.text_embedder.linear_1", H, cfg.pooled_dim, allow_fp8=False)
            self.p_out = f.linear("time_text_embed.text_embedder.linear_2", H, H)
        self.double: list[tuple[_StreamWeights, _StreamWeights]] = []
        self.single: list[_SingleWeights] = []
        for i in range(cfg.num_double_blocks):
            if not (self.block_range[0] <= i < self.block_range[1]):
                continue
            p = f"transformer_blocks.{i}."
            img = _StreamWeights(
                mod=lin_mod(p + "norm1.linear", 6),
                qkv=self._qkv(f, [p + "attn.to_q", p + "attn.to_k", p + "attn.to_v"]),
                q_norm=f.tensor(p + "attn.norm_q.weight", D, ones=True), k_norm=f.tensor(p + "attn.norm_k.weight", D, ones=True),
                proj=f.linear(p + "attn.to_out.0", H, cfg.num_heads * D, shard="row"),
                mlp_in=f.linear(p + "ff.net.0.proj", cfg.mlp_dim, H, shard="col"),
                mlp_out=f.linear(p + "ff.net.2", H, cfg.mlp_dim, shard="row"))
            txt = _StreamWeights(
                mod=lin_mod(p + "norm1_context.linear", 6),
                qkv=self._qkv(f, [p + "attn.add_q_proj", p + "attn.add_k_proj", p + "attn.add_v_proj"]),
                q_norm=f.tensor(p + "attn.norm_added_q.weight", D, ones=True),
                k_norm=f.tensor(p + "attn.norm_added_k.weight", D, ones=True),
                proj=f.linear(p + "attn.to_add_out", H, cfg.num_heads * D, shard="row"),
                mlp_in=f.linear(p + "ff_context.net.0.proj", cfg.mlp_dim, H, shard="col"),
                mlp_out=f.linear(p + "ff_context.net.2", H, cfg.mlp_dim, shard="row"))
            self.double.append(self._parked((img, txt), stream_blocks))
        for i in range(cfg.num_single_blocks):
            gi = cfg.num_double_blocks + i
            if not (self.block_range[0] <= gi < self.block_range[1]):
                continue
            p = f"single_transformer_blocks.{i}."
            self.single.append(self._parked(self._single(f, p), stream_blocks))
        if last and build_head:
            self.norm_out = lin_mod("norm_out.linear", 2)
            self.proj_out = f.linear("proj_out", cfg.latent_channels, H)
        if stream_blocks:
            self.enable_block_streaming()

    def _parked(self, block, stream_blocks: bool):
        if not stream_blocks or self.device.type != "cuda":
            return block
        from ...engine.block_streaming import map_tensors
        return map_tensors(block, lambda t: t.detach().cpu().pin_memory())

    # -- weight assembly ------------------------------------------------------------------
    def _qkv(self, f: WeightFactory, names) -> LinearWeight:
        """Fused [q_local; k_local; v_local] weight (each projection column-sharded by heads)."""
        H, D = self.cfg.hidden_size, self.cfg.head_dim
        parts = [f.linear(n, self.cfg.num_heads * D, H, shard="col", allow_fp8=False) for n in names]
        w = torch.cat([p.weight for p in parts], 0)
        b = torch.cat([p.bias for p in parts], 0) if parts[0].bias is not None else None
        return LinearWeight.from_dense(w, b, fp8=f.fp8 and w.is_cuda)

    def _single(self, f: WeightFactory, p: str) -> _SingleWeights:
        H, D, cfg = self.cfg.hidden_size, self.cfg.head_dim, self.cfg
        qkv = [f.linear(p + n, cfg.num_heads * D, H, shard="col", allow_fp8=False) for n in ("attn.to_q", "attn.to_k", "attn.to_v")]
        mlp = f.linear(p + "proj_mlp", cfg.mlp_dim, H, shard="col", allow_fp8=False)
        w = torch.cat([x.weight for x in qkv] + [mlp.weight], 0)
        b = torch.cat([x.bias for x in qkv] + [mlp.bias], 0)
        # proj_out consumes [attn (heads * D) | mlp]: shard each part of its input dim separately
        if f.get is not None:
            wo = f.get(p + "proj_out.weight")
            bo = f.get(p + "proj_out.bias")
        else:
            wo = f._rand(H, cfg.num_heads * D + cfg.mlp_dim)
            bo = f._rand(H)
        a_per, m_per = self.hl * D, self.mlp_l
        wo_a = wo[:, self.tp_rank * a_per:(self.tp_rank + 1) * a_per]
        wo_m = wo[:, cfg.num_heads * D + self.tp_rank * m_per: cfg.num_heads * D + (self.tp_rank + 1) * m_per]
        if self.tp_rank != 0:
            bo = torch.zeros_like(bo)
        out = LinearWeight.from_dense(torch.cat([wo_a, wo_m], 1).contiguous().to(self.device), bo.to(self.device),
                                      fp8=f.fp8 and self.device.type == "cuda")
        return _SingleWeights(mod=f.linear(p + "norm.linear", 3 * H, H) if self.HAS_MODULATION_LINEARS else None,
                              qkv_mlp=LinearWeight.from_dense(w, b, fp8=f.fp8 and w.is_cuda),
                              q_norm=f.tensor(p + "attn.norm_q.weight", D, ones=True),
                              k_norm=f.tensor(p + "attn.norm_k.weight", D, ones=True), out=out)

    def weight_bytes(self) -> int:
        n = 0
        for obj in [self.__dict__] + [b.__dict__ for pair in self.double for b in pair] + [s.__dict__ for s in self.single]:
            for v in obj.values():
                if isinstance(v, LinearWeight):
                    n += v.nbytes()
        return n

    # -- forward ---------------------------------------------------------------------------
    def _reduce(self, y: torch.Tensor) -> torch.Tensor:
        return self.comm.all_reduce(y) if self.tp > 1 else y

    def time_embedding(self, timestep: torch.Tensor, guidance: Optional[torch.Tensor], pooled: torch.Tensor) -> torch.Tensor:
        """temb [B, H] bf16 from sigma * 1000, guidance * 1000 and the pooled text vector."""
        dt = torch.bfloat16
        te = timestep_embedding(timestep * 1000.0, 256).to(dt)
        temb = ops.linear(ops.linear(te, self.t_in, act="silu"), self.t_out).float()
        if self.cfg.guidance_embed and guidance is not None:
            ge = timestep_embedding(guidance * 1000.0, 256).to(dt)
            temb = temb + ops.linear(ops.linear(ge, self.g_in, act="silu"), self.g_out).float()
        temb = temb + ops.linear(ops.linear(pooled.to(dt), self.p_in, act="silu"), self.p_out).float()
        return temb.to(dt)

    def enable_block_streaming(self) -> None:
        """Keep the transformer blocks in pinned host memory and stream them through two device
        slots during the forward pass (low-VRAM mode; see engine/block_streaming.py)."""
        from ...engine.block_streaming import BlockStreamer
        self._streamers = {"double": BlockStreamer(self.double, self.device), "single": BlockStreamer(self.single, self.device)}
        # the resident copies are dropped: the streamer owns the (host) weights now
        self.double = [None] * len(self.double)
        self.single = [None] * len(self.single)

    def _blocks(self, blocks, kind: str):
        st = getattr(self, "_streamers", None)
        if not st:
            yield from blocks
            return
        s = st[kind]
        s.prime()
        for i in range(len(s)):
            yield s.block(i)
        s.evict_all()

    def _mod(self, temb_act: torch.Tensor, w, kind: str, index: int) -> torch.Tensor:
        """AdaLN vectors of one block: ``kind`` is "img" / "txt" (double block ``index``) or "single".
        Flux computes them from the time / text embedding; variants that look them up override this."""
        return modulation(temb_act, w)

    def _final_mod(self, temb_act: torch.Tensor) -> torch.Tensor:
        return ops.linear(temb_act, self.norm_out)

    def _attend(self, q, k, v, batch: int) -> torch.Tensor:
        """q, k, v [B * S, Hl, D] -> [B * S, Hl * D]; one attention call per sample."""
        s = q.shape[0] // batch
        outs = [ops.attention(q[b * s:(b + 1) * s], k[b * s:(b + 1) * s], v[b * s:(b + 1) * s]) for b in range(batch)]
        o = outs[0] if batch == 1 else torch.cat(outs, 0)
        return o.reshape(o.shape[0], -1)

    def _gated_add(self, x, y, gate, rows_per_batch):
        return ops.gated_residual(x, y, gate, rows_per_batch)

    def _fused_rows(self, tokens: int):
        """The fused GEMM + all-reduce + gated residual kernel (parallel/fused.py, large-token form)
        sized for ``tokens`` rows, or None (one rank, CPU, flag off, no peer mapping)."""
        if self.tp == 1 or self.device.type != "cuda" or not config.get("fused_dit_tp"):
            return None
        cur = getattr(self, "_fused_rp", None)
        if cur is None or (cur is not False and cur.max_large_tokens < tokens):
            from ...parallel.fused import FusedRowParallel
            try:
                if cur:
                    cur.close()
                self._fused_rp = FusedRowParallel(self.comm, self.cfg.hidden_size, self.device, max_large_tokens=tokens)
                self.comm_path = "fused GEMM + all-reduce + gated residual (multimem)" if self._fused_rp.use_mc else \
                    "fused GEMM + all-reduce + gated residual (peer loads)"
            except Exception as e:
                log.warn(f"[TensorParallel] fused row-parallel kernel unavailable ({type(e).__name__}: {e}); using NCCL")
                self._fused_rp = False
        return self._fused_rp or None

    def _fused_cols(self, tokens: int):
        """The all-gather -> GEMM kernel (parallel/fused.py) for ``tokens`` rows of width H, or None."""
        cur = getattr(self, "_fused_cp", None)
        if cur is None or (cur is not False and cur.max_tokens < tokens):
            from ...parallel.fused import FusedColumnParallel
            try:
                if cur:
                    cur.close()
                self._fused_cp = FusedColumnParallel(self.comm, tokens, self.cfg.hidden_size, self.device)
            except Exception as e:
                log.warn(f"[TensorParallel] all-gather GEMM kernel unavailable ({type(e).__name__}: {e})")
                self._fused_cp = False
        return self._fused_cp or None

    def close(self) -> None:
        for name in ("_fused_rp", "_fused_cp"):
            cur = getattr(self, name, None)
            if cur:
                cur.close()
            setattr(self, name, None)

    def _forward_sp(self, img, txt, timestep, pooled, img_ids, txt_ids, guidance, rp, cp):
        """Sequence-parallel form of :meth:`forward` for one sample on a tensor-parallel group: between
        the row-parallel and the column-parallel linears every rank keeps only its block of token
        rows, so norms, modulations, gated residuals and activation quantisation run on 1 / tp of the
        rows. Row-parallel linears end in a reduce-scatter inside the GEMM kernel (``rp.large`` with
        ``scatter_out``), column-parallel linears start with an all-gather inside the GEMM kernel
        (``cp``). Attention sees all tokens of the rank's heads, as before."""
        cfg = self.cfg
        S_i, S_t = img.shape[1], txt.shape[1]
        S = S_t + S_i
        H, D = cfg.hidden_size, cfg.head_dim
        dt = torch.bfloat16
        temb = self.time_embedding(timestep, guidance, pooled)
        temb_act = silu(temb)
        cos, sin = rope_tables(torch.cat([txt_ids, img_ids], 0).to(self.device), cfg.axes_dim, cfg.theta)
        cos_t, sin_t, cos_i, sin_i = cos[:S_t].contiguous(), sin[:S_t].contiguous(), cos[S_t:].contiguous(), sin[S_t:].contiguous()
        (ai, bi_), (at, bt_) = rp.owned_rows(S_i), rp.owned_rows(S_t)
        x_i = ops.linear(img.reshape(S_i, -1)[ai:bi_].to(dt).contiguous(), self.x_embedder)        # the rank's image rows
        x_t = ops.linear(txt.reshape(S_t, -1)[at:bt_].to(dt).contiguous(), self.context_embedder)  # the rank's text rows

        def pre(x, w, mod, rows_total, c, s_):
            xn, _, xq = ops.norm(x, None, shift=mod[:, 0:H], scale=mod[:, H:2 * H], rows_per_batch=x.shape[0], layernorm=True,
                                 emit_fp8=self.fp8 and w.qkv.is_fp8, emit_bf16=not (self.fp8 and w.qkv.is_fp8))
            qkv = cp(xq if xq is not None else xn, w.qkv, rows_total)
            return ops.dit_qkv(qkv, self.hl, self.hl, D, q_norm_w=w.q_norm, k_norm_w=w.k_norm, cos=c, sin=s_)

        def post(x, a, w, mod, rows_total):
            x = rp.large(a, w.proj, res=x, gate=mod[0, 2 * H:3 * H].contiguous(), scatter_out=torch.empty_like(x))
            xn, _, xq = ops.norm(x, None, shift=mod[:, 3 * H:4 * H], scale=mod[:, 4 * H:5 * H], rows_per_batch=x.shape[0],
                                 layernorm=True, emit_fp8=self.fp8 and w.mlp_in.is_fp8,
                                 emit_bf16=not (self.fp8 and w.mlp_in.is_fp8))
            h = cp(xq if xq is not None else xn, w.mlp_in, rows_total, act="gelu_tanh")
            return rp.large(h, w.mlp_out, res=x, gate=mod[0, 5 * H:6 * H].contiguous(), scatter_out=torch.empty_like(x))

        for bi, (wi, wt) in enumerate(self._blocks(self.double, "double")):
            mod_i, mod_t = self._mod(temb_act, wi.mod, "img", bi), self._mod(temb_act, wt.mod, "txt", bi)
            qi, ki, vi = pre(x_i, wi, mod_i, S_i, cos_i, sin_i)
            qt, kt, vt = pre(x_t, wt, mod_t, S_t, cos_t, sin_t)
            att = self._attend(torch.cat([qt, qi], 0), torch.cat([kt, ki], 0), torch.cat([vt, vi], 0), 1)
            x_i = post(x_i, att[S_t:].contiguous(), wi, mod_i, S_i)
            x_t = post(x_t, att[:S_t].contiguous(), wt, mod_t, S_t)

        # the single blocks work on the joint sequence [txt | img], cut into blocks of rows again
        def gather_rows(x, rows_total):
            per = (rows_total + self.tp - 1) // self.tp
            pad = torch.zeros(per, H, dtype=dt, device=self.device)
            pad[:x.shape[0]] = x
            return self.comm.all_gather(pad, dim=0)[:rows_total]

        aj, bj = rp.owned_rows(S)
        if self.single:
            joint = torch.cat([gather_rows(x_t, S_t), gather_rows(x_i, S_i)], 0)[aj:bj].contiguous()
            qkv_cols = 3 * self.hl * D
            for si, w in enumerate(self._blocks(self.single, "single")):
                mod = self._mod(temb_act, w.mod, "single", si)
                xn, _, xq = ops.norm(joint, None, shift=mod[:, 0:H], scale=mod[:, H:2 * H], rows_per_batch=joint.shape[0],
                                     layernorm=True, emit_fp8=self.fp8 and w.qkv_mlp.is_fp8,
                                     emit_bf16=not (self.fp8 and w.qkv_mlp.is_fp8))
                fused = cp(xq if xq is not None else xn, w.qkv_mlp, S)                       # [S, 3 Hl D + mlp_l]
                q, k, v = ops.dit_qkv(fused[:, :qkv_cols], self.hl, self.hl, D, q_norm_w=w.q_norm, k_norm_w=w.k_norm,
                                      cos=cos, sin=sin)
                att = self._attend(q, k, v, 1)
                mlp = torch.nn.functional.gelu(fused[:, qkv_cols:].float(), approximate="tanh").to(dt)
                joint = rp.large(torch.cat([att, mlp], 1), w.out, res=joint, gate=mod[0, 2 * H:3 * H].contiguous(),
                                 scatter_out=torch.empty_like(joint))
            x_img = gather_rows(joint, S)[S_t:]
        else:
            x_img = gather_rows(x_i, S_i)
        mo = self._final_mod(temb_act)
        xn, _, _ = ops.norm(x_img.contiguous(), None, shift=mo[:, H:2 * H], scale=mo[:, 0:H], rows_per_batch=S_i, layernorm=True)
        out = ops.linear(xn, self.proj_out)
        return out.reshape(1, S_i, cfg.latent_channels)

    def _row_parallel(self, a, w, x, gate, rows_per_batch, fused, slot):
        """x + gate * all_reduce(a w^T + bias): one fused kernel where it applies."""
        if fused is not None and gate.shape[0] == 1 and fused.supports_large(a.shape[0], w.weight.shape[0]):
            return fused.large(a, w, res=x.contiguous(), gate=gate.reshape(-1).contiguous(), slot=slot)
        return self._gated_add(x, self._reduce(ops.linear(a, w)), gate, rows_per_batch)

    def forward(self, img: torch.Tensor, txt: torch.Tensor, timestep: torch.Tensor, pooled: torch.Tensor,
                img_ids: torch.Tensor, txt_ids: torch.Tensor, guidance: Optional[torch.Tensor] = None,
                hidden_in: Optional[tuple] = None, step_cache=None, control: Optional[tuple] = None,
                collect: Optional[tuple] = None):
        """img [B, S_i, C_in] packed latents, txt [B, S_t, context_dim], timestep (sigma) [B],
        pooled [B, pooled_dim], ids [S, 3]. Returns the velocity prediction [B, S_i, C_in] (bf16), or
        the (img, txt | joint) hidden state when this instance holds only a block range.
        ``step_cache`` (a :class:`~.step_cache.FirstBlockCache`, whole-model instances only): after the
        first block decide whether the rest of the stack can be replaced by last step's residual.
        ``control`` = (double residuals, single residuals): lists of [B * S_i, H] tensors from a
        ControlNet, added to the image stream after the blocks they map to (one residual covers
        ceil(blocks / residuals) consecutive blocks). ``collect`` = (list, list): filled with the image
        stream after every double / single block (what a ControlNet branch projects)."""
        cfg = self.cfg
        B, S_i = img.shape[0], img.shape[1]
        S_t = txt.shape[1]
        H, D = cfg.hidden_size, cfg.head_dim
        dt = torch.bfloat16
        if (self.tp > 1 and B == 1 and hidden_in is None and step_cache is None and control is None and collect is None
                and self.has_head and self.block_range == (0, cfg.num_double_blocks + cfg.num_single_blocks)
                and min(S_i, S_t) > 128 and not getattr(self, "_streamers", None) and config.get("fused_dit_sp")):
            rp = self._fused_rows(S_i + S_t)
            cp = self._fused_cols(S_i + S_t) if rp is not None else None
            if rp is not None and cp is not None:
                self.comm_path = ("sequence-parallel blocks: all-gather -> GEMM and GEMM -> reduce-scatter kernels ("
                                  + ("multimem" if rp.use_mc else "peer loads") + ")")
                return self._forward_sp(img, txt, timestep, pooled, img_ids, txt_ids, guidance, rp, cp)
        temb = self.time_embedding(timestep, guidance, pooled)
        temb_act = silu(temb)
        cos, sin = rope_tables(torch.cat([txt_ids, img_ids], 0).to(self.device), cfg.axes_dim, cfg.theta)
        cos_t, sin_t, cos_i, sin_i = cos[:S_t].contiguous(), sin[:S_t].contiguous(), cos[S_t:].contiguous(), sin[S_t:].contiguous()
        if B > 1:
            cos_t, sin_t, cos_i, sin_i = (x.repeat(B, 1) for x in (cos_t, sin_t, cos_i, sin_i))
        if hidden_in is None:
            x_i = ops.linear(img.reshape(B * S_i, -1).to(dt), self.x_embedder)
            x_t = ops.linear(txt.reshape(B * S_t, -1).to(dt), self.context_embedder)
            joint = None
        else:
            x_i, x_t, joint = hidden_in

        def stream_pre(x, w: _StreamWeights, mod, S, c, s):
            xn, _, xq = ops.norm(x, None, shift=mod[:, 0:H], scale=mod[:, H:2 * H], rows_per_batch=S, layernorm=True,
                                 emit_fp8=self.fp8 and w.qkv.is_fp8, emit_bf16=not (self.fp8 and w.qkv.is_fp8))
            qkv = ops.linear(xq if xq is not None else xn, w.qkv)
            return ops.dit_qkv(qkv, self.hl, self.hl, D, q_norm_w=w.q_norm, k_norm_w=w.k_norm, cos=c, sin=s)

        # the fused row-parallel kernel hands out views of its own buffers: not while something
        # (ControlNet residual collection, the step cache) keeps the streams beyond the next block
        rp_fused = self._fused_rows(B * (S_i + S_t)) if (control is None and collect is None and step_cache is None) else None

        def stream_post(x, a, w: _StreamWeights, mod, S, slot):
            x = self._row_parallel(a, w.proj, x, mod[:, 2 * H:3 * H], S, rp_fused, slot)
            xn, _, xq = ops.norm(x, None, shift=mod[:, 3 * H:4 * H], scale=mod[:, 4 * H:5 * H], rows_per_batch=S,
                                 layernorm=True, emit_fp8=self.fp8 and w.mlp_in.is_fp8,
                                 emit_bf16=not (self.fp8 and w.mlp_in.is_fp8))
            h = ops.linear(xq if xq is not None else xn, w.mlp_in, act="gelu_tanh")
            return self._row_parallel(h, w.mlp_out, x, mod[:, 5 * H:6 * H], S, rp_fused, slot + 1)

        whole = self.block_range == (0, cfg.num_double_blocks + cfg.num_single_blocks)
        use_cache = step_cache is not None and step_cache.enabled and whole and len(self.double) > 0
        first_x_i = None
        skip_rest = False
        for bi, (wi, wt) in enumerate(self._blocks(self.double, "double")):
            if skip_rest:
                break
            mod_i, mod_t = self._mod(temb_act, wi.mod, "img", self.block_range[0] + bi), self._mod(temb_act, wt.mod, "txt", self.block_range[0] + bi)
            qi, ki, vi = stream_pre(x_i, wi, mod_i, S_i, cos_i, sin_i)
            qt, kt, vt = stream_pre(x_t, wt, mod_t, S_t, cos_t, sin_t)
            # joint sequence per sample: [txt | img]
            def join(a, b):
                if B == 1:
                    return torch.cat([a, b], 0)
                return torch.cat([torch.cat([a[i * S_t:(i + 1) * S_t], b[i * S_i:(i + 1) * S_i]], 0) for i in range(B)], 0)
            att = self._attend(join(qt, qi), join(kt, ki), join(vt, vi), B)
            S = S_t + S_i
            if B == 1:
                a_t, a_i = att[:S_t], att[S_t:]
            else:
                a_t = torch.cat([att[i * S:i * S + S_t] for i in range(B)], 0)
                a_i = torch.cat([att[i * S + S_t:(i + 1) * S] for i in range(B)], 0)
            x_i = stream_post(x_i, a_i.contiguous(), wi, mod_i, S_i, 0)
            x_t = stream_post(x_t, a_t.contiguous(), wt, mod_t, S_t, 2)
            if collect is not None:
                collect[0].append(x_i)
            if control is not None and control[0]:
                every = -(-cfg.num_double_blocks // len(control[0]))
                x_i = (x_i.float() + control[0][(self.block_range[0] + bi) // every].float()).to(dt)
            if use_cache and bi == 0:
                first_x_i = x_i
                if not step_cache.should_compute(x_i):
                    x_i = step_cache.apply_residual(x_i)
                    skip_rest = True

        if not skip_rest and (self.single or self.block_range[1] > cfg.num_double_blocks):
            S = S_t + S_i
            if joint is None:
                if B == 1:
                    joint = torch.cat([x_t, x_i], 0)
                else:
                    joint = torch.cat([torch.cat([x_t[i * S_t:(i + 1) * S_t], x_i[i * S_i:(i + 1) * S_i]], 0) for i in range(B)], 0)
            cj, sj = (cos, sin) if B == 1 else (cos.repeat(B, 1), sin.repeat(B, 1))
            qkv_cols = 3 * self.hl * D
            for si, w in enumerate(self._blocks(self.single, "single")):
                mod = self._mod(temb_act, w.mod, "single", si)
                xn, _, xq = ops.norm(joint, None, shift=mod[:, 0:H], scale=mod[:, H:2 * H], rows_per_batch=S, layernorm=True,
                                     emit_fp8=self.fp8 and w.qkv_mlp.is_fp8, emit_bf16=not (self.fp8 and w.qkv_mlp.is_fp8))
                fused = ops.linear(xq if xq is not None else xn, w.qkv_mlp)     # [T, 3 Hl D + mlp_l]
                q, k, v = ops.dit_qkv(fused[:, :qkv_cols], self.hl, self.hl, D, q_norm_w=w.q_norm, k_norm_w=w.k_norm,
                                      cos=cj, sin=sj)
                att = self._attend(q, k, v, B)
                mlp = torch.nn.functional.gelu(fused[:, qkv_cols:].float(), approximate="tanh").to(dt)
                joint = self._row_parallel(torch.cat([att, mlp], 1), w.out, joint, mod[:, 2 * H:3 * H], S, rp_fused, si & 1)
                if collect is not None or (control is not None and control[1]):
                    img_rows = slice(S_t, S) if B == 1 else None
                    if img_rows is None:
                        raise ValueError("ControlNet residuals on the single blocks need batch 1")
                    if collect is not None:
                        collect[1].append(joint[img_rows])
                    if control is not None and control[1]:
                        every = -(-cfg.num_single_blocks // len(control[1]))
                        joint = joint.clone()
                        joint[img_rows] = (joint[img_rows].float() + control[1][si // every].float()).to(dt)
            if self.block_range[1] == cfg.num_double_blocks + cfg.num_single_blocks:
                if B == 1:
                    x_i = joint[S_t:]
                else:
                    x_i = torch.cat([joint[i * S + S_t:(i + 1) * S] for i in range(B)], 0)
        if self.block_range[1] != cfg.num_double_blocks + cfg.num_single_blocks or not self.has_head:
            return x_i, x_t, joint
        if use_cache and not skip_rest:
            step_cache.store_residual(first_x_i, x_i)
        mo = self._final_mod(temb_act)                                        # [B, 2H]: scale, shift
        xn, _, _ = ops.norm(x_i.contiguous(), None, shift=mo[:, H:2 * H], scale=mo[:, 0:H], rows_per_batch=S_i, layernorm=True)
        out = ops.linear(xn, self.proj_out)
        return out.reshape(B, S_i, cfg.latent_channels)


def flux_ids(height_tokens: int, width_tokens: int, text_tokens: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """Position ids: image tokens get (0, y, x), text tokens (0, 0, 0)."""
    ys, xs = torch.meshgrid(torch.arange(height_tokens), torch.arange(width_tokens), indexing="ij")
    img = torch.stack([torch.zeros_like(ys), ys, xs], -1).reshape(-1, 3).to(device)
    txt = torch.zeros(text_tokens, 3, dtype=img.dtype, device=device)
    return img, txt
