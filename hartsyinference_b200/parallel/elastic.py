"""Failure detection and regrouping of a rank group, on the host.

Every rank publishes a heartbeat (a counter and a wall-clock stamp) into a key-value store that
rank 0 serves (``torch.distributed.TCPStore``); between steps, before it launches anything that
waits on a peer, a rank asks which peers have gone quiet. When some have, the survivors drop the
old process group and form a new, smaller one over the same store (a fresh key prefix per
generation), after which the caller re-shards its model for the lower degree and carries on.

A rank only ever leaves between steps, with none of its kernels or collectives in flight; the
others learn of it here, on the host, before their next launch. Inside kernels the bounded waits
(``csrc/kernels/common.cuh``) remain the backstop: a peer that disappears mid-step makes the wait
run out, the status word reports it, and the engine fails that step's requests and falls back to
NCCL or regroups through this module.

The reference has no multi-process group to lose: its only cross-device rendezvous is the
context-parallel K/V exchange, a timed barrier with an abort flag
(src/HartsyInference.Diffusion/Utilities/CpKvExchange.cs:41-135), and its scheduler contains step
faults by failing the step's requests (src/HartsyInference.LLM/Generation/DynamicBatchScheduler.cs:
125-145); both behaviours are kept (bounded waits; ``LLMEngine.step``'s fault containment).
"""
from __future__ import annotations

import datetime
import time
from typing import Optional, Sequence

from .. import log
from ..exceptions import CommError
from .comm import Comm, SingleComm, TorchDistComm


class ElasticGroup:
    """``world`` ranks sharing a TCP store on ``host:port`` (rank 0 hosts it). Use::

        eg = ElasticGroup(rank, world, "127.0.0.1", port, backend="gloo")
        comm = eg.comm                      # TorchDistComm over all ranks
        ... step ...
        eg.beat()
        dead = eg.dead(timeout_s=2.0)
        if dead:
            comm = eg.regroup([r for r in range(world) if r not in dead])
    """

    def __init__(self, rank: int, world: int, host: str, port: int, backend: str = "gloo",
                 timeout_s: float = 30.0):
        import torch.distributed as dist
        self._dist = dist
        self.rank0, self.world0 = rank, world            # identity in the original numbering
        self.members = list(range(world))                # original ranks of the current group
        self.backend = backend
        self.timeout = datetime.timedelta(seconds=timeout_s)
        self.store = dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=self.timeout,
                                   wait_for_workers=True)
        self.generation = 0
        self._beats = 0
        self.comm: Comm = self._init_group()
        self.beat()

    # ------------------------------------------------------------------ group (re)creation
    def _init_group(self) -> Comm:
        dist = self._dist
        if len(self.members) == 1:
            return SingleComm()
        store = dist.PrefixStore(f"gen{self.generation}", self.store)
        dist.init_process_group(self.backend, store=store, rank=self.members.index(self.rank0),
                                world_size=len(self.members), timeout=self.timeout)
        log.decision("Collective", f"group generation {self.generation}: ranks {self.members} "
                                   f"(this is original rank {self.rank0}) transport={self.backend}")
        return TorchDistComm()

    def regroup(self, survivors: Sequence[int]) -> Comm:
        """Called by every surviving rank with the same list of original ranks. Tears the old group
        down without waiting for the lost ranks and builds the next generation."""
        survivors = sorted(int(r) for r in survivors)
        if self.rank0 not in survivors:
            raise CommError(f"rank {self.rank0} is not among the survivors {survivors}")
        if 0 not in survivors:
            raise CommError("rank 0 hosts the store; the group cannot outlive it")
        if self._dist.is_initialized():
            try:
                self._dist.destroy_process_group()
            except Exception as e:      # a dead peer can make the teardown complain; the group is gone either way
                log.warn(f"[Collective] teardown of generation {self.generation}: {type(e).__name__}: {e}")
        self.members = survivors
        self.generation += 1
        self.comm = self._init_group()
        return self.comm

    # ------------------------------------------------------------------ heartbeats
    def beat(self) -> None:
        """Publish "alive" (call between steps)."""
        self._beats += 1
        self.store.set(f"hb/{self.rank0}", f"{self._beats}:{time.time():.3f}")

    def leave(self) -> None:
        """Announce an orderly departure (between steps) so that peers need not wait for a timeout."""
        self.store.set(f"hb/{self.rank0}", "left")

    def last_seen(self, rank: int) -> Optional[float]:
        """Wall-clock time of ``rank``'s last heartbeat; None when it left or never reported."""
        try:
            if not self.store.check([f"hb/{rank}"]):
                return None
            raw = self.store.get(f"hb/{rank}").decode()
        except Exception:
            return None
        if raw == "left":
            return None
        return float(raw.split(":")[1])

    def dead(self, timeout_s: float = 2.0) -> list[int]:
        """Members (original ranks) whose last heartbeat is older than ``timeout_s`` or who left."""
        now = time.time()
        out = []
        for r in self.members:
            if r == self.rank0:
                continue
            seen = self.last_seen(r)
            if seen is None or now - seen > timeout_s:
                out.append(r)
        return out

    def agree_on_survivors(self, timeout_s: float = 2.0) -> list[int]:
        """Rank 0 decides who is still there and publishes the list for this generation; the other
        survivors read it (so that all of them regroup with the same membership)."""
        key = f"survivors/{self.generation}"
        if self.rank0 == 0:
            lost = set(self.dead(timeout_s))
            alive = [r for r in self.members if r not in lost]
            self.store.set(key, ",".join(str(r) for r in alive))
            return alive
        self.store.wait([key], self.timeout)
        return [int(x) for x in self.store.get(key).decode().split(",") if x]

    def close(self) -> None:
        if self._dist.is_initialized():
            try:
                self._dist.destroy_process_group()
            except Exception:
                pass
