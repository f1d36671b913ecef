"""SPMD execution of the engine over several GPUs: one process per GPU (``torch.distributed.run``),
every process builds the same ``InferenceEngine``; rank 0 is the front (the API caller, the HTTP
server, the CLI) and the other ranks follow it.

The reference drives all of its devices from one process: ``InferenceEngine.EnsureBackend`` /
``EnsureCfgParallelBackend`` / ``EnsureDitShardBackends`` / ``EnsureCpBackends`` create one backend
object per ordinal (src/HartsyInference.Engine/InferenceEngine.cs:198-208) and ``TextService.
LoadTensorParallel`` / ``LoadSharded`` slice a model over them (Services/TextService.cs:271-280,
406-506). Here each device has its own process, so the same decisions become process groups:

* :class:`RankContext` reads the torchrun environment, opens the world communicator (NCCL on GPUs,
  gloo on CPU ranks) plus a gloo group for small Python objects, and carves the groups a
  :class:`~hartsyinference_b200.parallel.config.ParallelConfig` asks for: ranks are ordered
  ``[dp][cfg][tp * sp]``; the innermost group is the tensor- or sequence-parallel group, ``cfg`` pairs
  rank i of the conditional group with rank i of the unconditional group.
* Commands: whatever rank 0 does that needs the other ranks (load a model, run one scheduler tick,
  denoise an image) is first broadcast as a small tuple; followers sit in :meth:`follow` and run the
  same call, so the collectives inside the model code line up. One lock on rank 0 keeps commands
  from different API threads in one order.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from .. import log
from ..exceptions import CommError
from ..parallel.comm import Comm, SingleComm, TorchDistComm, init_comm
from ..parallel.config import ParallelConfig


@dataclass
class ParallelGroups:
    inner: Comm                 # tensor-parallel (LLM, image DiT) or sequence-parallel (video DiT) group
    cfg: Optional[Comm]         # 2-rank group pairing the guidance branches, or None
    dp_index: int               # which replica this rank belongs to
    dp: int
    inner_rank: int
    cfg_index: int


class RankContext:
    """The process group an engine instance lives in. ``RankContext.from_env()`` returns None for a
    single process."""

    def __init__(self, world: Comm):
        import torch.distributed as dist
        self._dist = dist
        self.world = world
        self.rank, self.size = world.rank, world.world
        # small Python objects travel over gloo: no device synchronisation, no GPU staging
        self.control = dist.new_group(backend="gloo") if dist.get_backend() != "gloo" else None
        self.lock = threading.RLock()            # rank 0: orders commands issued by different threads
        self._groups: dict[str, ParallelGroups] = {}
        self._handlers: dict[str, Callable[..., Any]] = {}
        self._following = False
        # a follower whose handler raised says so here; rank 0 looks before every command, so that a
        # rank that fell out of step ends the next call with an error instead of a hung collective
        try:
            self._store = dist.distributed_c10d._get_default_store()
        except Exception:
            self._store = None

    @staticmethod
    def from_env() -> Optional["RankContext"]:
        if int(os.environ.get("WORLD_SIZE", "1")) <= 1:
            return None
        comm = init_comm()
        if comm.world <= 1:
            return None
        return RankContext(comm)

    @property
    def is_front(self) -> bool:
        return self.rank == 0

    # ---------------------------------------------------------------------------- objects
    def broadcast(self, obj: Any = None) -> Any:
        """Rank 0's ``obj`` on every rank (all ranks call this together)."""
        box = [obj if self.rank == 0 else None]
        self._dist.broadcast_object_list(box, src=0, group=self.control)
        return box[0]

    def gather(self, obj: Any) -> Optional[list]:
        """Every rank's ``obj`` as a list on rank 0 (None elsewhere)."""
        out = [None] * self.size if self.rank == 0 else None
        self._dist.gather_object(obj, out, dst=0, group=self.control)
        return out

    # ---------------------------------------------------------------------------- groups
    def groups(self, placement: ParallelConfig) -> ParallelGroups:
        """Process groups for a placement (cached per placement; every rank must ask for the same
        placements in the same order, which the command stream guarantees)."""
        key = placement.cache_key
        got = self._groups.get(key)
        if got is not None:
            return got
        inner_n = max(1, placement.tp) * max(1, placement.sp)
        if placement.tp > 1 and placement.sp > 1:
            raise CommError("tensor and sequence parallelism cannot be combined in one group")
        if placement.pp > 1:
            raise CommError("pipeline stages are driven by parallel.pipeline.PipelinedModel, not by the SPMD services")
        cfg_n = 2 if placement.cfg == 2 else 1
        need = inner_n * cfg_n
        if self.size % need != 0:
            raise CommError(f"placement {placement.describe()} needs a multiple of {need} ranks, {self.size} are running")
        dp = self.size // need
        if placement.dp not in (1, dp):
            raise CommError(f"placement {placement.describe()} asks for dp={placement.dp}; {self.size} ranks give dp={dp}")
        world = self.world
        assert isinstance(world, TorchDistComm)
        mine_inner: Comm = SingleComm()
        mine_cfg: Optional[Comm] = None
        # every rank creates every group, in the same order
        for d in range(dp):
            for c in range(cfg_n):
                ranks = [(d * cfg_n + c) * inner_n + i for i in range(inner_n)]
                if inner_n > 1:
                    g = world.subgroup(ranks)
                    if self.rank in ranks:
                        mine_inner = g
            if cfg_n == 2:
                for i in range(inner_n):
                    pair = [(d * 2) * inner_n + i, (d * 2 + 1) * inner_n + i]
                    g = world.subgroup(pair)
                    if self.rank in pair:
                        mine_cfg = g
        blk = self.rank // inner_n
        out = ParallelGroups(inner=mine_inner, cfg=mine_cfg, dp_index=blk // cfg_n, dp=dp,
                             inner_rank=self.rank % inner_n, cfg_index=blk % cfg_n)
        self._groups[key] = out
        log.decision("Placement", f"rank {self.rank}/{self.size}: {placement.describe()} -> replica {out.dp_index} of {dp}, "
                                  f"inner rank {out.inner_rank}/{inner_n}" + (f", cfg branch {out.cfg_index}" if cfg_n == 2 else ""))
        return out

    # ---------------------------------------------------------------------------- commands
    def register(self, name: str, fn: Callable[..., Any]) -> None:
        self._handlers[name] = fn

    def command(self, name: str, *args: Any) -> Any:
        """Rank 0: tell the followers to run handler ``name`` with ``args``, then run it here too and
        return its result. Must not be called on followers."""
        if self.rank != 0:
            raise CommError("commands are issued by rank 0 only")
        with self.lock:
            failed = self.follower_failure()
            if failed:
                raise CommError(f"a follower rank fell out of step: {failed}")
            self.broadcast((name, args))
            return self._handlers[name](*args)

    def follower_failure(self) -> Optional[str]:
        """What a follower reported when one of its command handlers raised (None: all in step)."""
        if self._store is None:
            return None
        try:
            if self._store.check(["spmd/failed"]):
                return self._store.get("spmd/failed").decode()
        except Exception:
            return None
        return None

    def follow(self) -> None:
        """Followers: run rank 0's commands until it sends ``shutdown``."""
        if self.rank == 0:
            return
        self._following = True
        while True:
            name, args = self.broadcast()
            if name == "shutdown":
                break
            try:
                self._handlers[name](*args)
            except Exception as e:      # keep following: rank 0 sees its own copy of the failure
                log.warn(f"[Placement] follower rank {self.rank}: command {name} failed: {type(e).__name__}: {e}")
                if self._store is not None:
                    try:
                        self._store.set("spmd/failed", f"rank {self.rank}, command {name}: {type(e).__name__}: {e}")
                    except Exception:
                        pass
        self._following = False

    def shutdown(self) -> None:
        """Rank 0: release the followers."""
        if self.rank == 0 and self.size > 1:
            with self.lock:
                self.broadcast(("shutdown", ()))

    def ready_report(self, ok: bool) -> Optional[list]:
        """Collective health probe: every rank's flag on rank 0 (issued through :meth:`command`)."""
        return self.gather(bool(ok))
