"""Collective communication front end.

``Comm`` is the small interface the models call (all_reduce / all_gather / reduce_scatter /
all_to_all / send / recv / barrier). Implementations:

* ``SingleComm``     world size 1, every op is the identity;
* ``TorchDistComm``  ``torch.distributed`` process group: NCCL on GPUs (the measured baseline of
  every fused path and the transport of pipeline send/recv) or gloo for CPU ranks in tests;
* ``FusedComm`` (:mod:`.fused`) adds the hand-written NVLink kernels on top of a TorchDistComm.

The reference's counterpart is ``ICollectiveComm`` with two ops (AllReduceSum, AllGather;
src/HartsyInference.Core/Backends/ICollectiveComm.cs:12-28), an NCCL implementation driven from
one process (src/HartsyInference.Cuda/NcclComm.cs:53-121) and a host-staged fp32 fallback
(src/HartsyInference.Core/Backends/HostStagedComm.cs:32-79); the selection ladder of
``CollectiveComm.Create`` (src/HartsyInference.Cuda/CollectiveComm.cs:12-58) is mirrored by
:func:`init_comm`, including its ``[Collective] transport=...`` log line.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional, Sequence

import torch

from .. import log


class Comm:
    rank: int = 0
    world: int = 1
    transport: str = "single"

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return t

    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return t

    def all_to_all(self, t: torch.Tensor, split_dim: int, concat_dim: int) -> torch.Tensor:
        return t

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        return t

    def send(self, t: torch.Tensor, dst: int) -> None:
        raise RuntimeError("send on a single-rank communicator")

    def recv(self, t: torch.Tensor, src: int) -> torch.Tensor:
        raise RuntimeError("recv on a single-rank communicator")

    def isend(self, t: torch.Tensor, dst: int):
        raise RuntimeError("isend on a single-rank communicator")

    def irecv(self, t: torch.Tensor, src: int):
        raise RuntimeError("irecv on a single-rank communicator")

    def barrier(self) -> None:
        return None

    def all_gather_object(self, obj):
        return [obj]


class SingleComm(Comm):
    pass


class ShardEmulationComm(Comm):
    """Measurement aid: claims to be ``rank`` of ``world`` but has no peers. Models built on it
    hold exactly one rank's weight shard and run that rank's kernels; every collective returns its
    input, so the OUTPUTS ARE NOT MEANINGFUL. It exists to time one rank's compute of a TP / EP
    layout on a single GPU (the collectives' cost has to be added from a multi-GPU run)."""
    transport = "emulated-shard"

    def __init__(self, world: int, rank: int = 0):
        self.world, self.rank = world, rank


class TorchDistComm(Comm):
    """A (sub)group of the default ``torch.distributed`` world."""

    def __init__(self, group=None, ranks: Optional[Sequence[int]] = None):
        import torch.distributed as dist
        self._dist = dist
        self.group = group
        self.ranks = list(ranks) if ranks is not None else list(range(dist.get_world_size()))
        self.world = len(self.ranks)
        self.global_rank = dist.get_rank()
        self.rank = self.ranks.index(self.global_rank)
        self.transport = dist.get_backend(group)

    def all_reduce(self, t):
        self._dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t, dim=0):
        t = t.contiguous()
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self._dist.all_gather_into_tensor(out, t, group=self.group) if t.is_cuda else \
            self._dist.all_gather(list(out.unbind(0)), t, group=self.group)
        if dim == 0:
            return out.reshape((-1,) + tuple(t.shape[1:]))
        return torch.cat(list(out.unbind(0)), dim=dim)

    def reduce_scatter(self, t, dim=0):
        chunks = [c.contiguous() for c in t.chunk(self.world, dim=dim)]
        out = torch.empty_like(chunks[0])
        if t.is_cuda:
            self._dist.reduce_scatter(out, chunks, group=self.group)
        else:  # gloo has no reduce_scatter
            full = t.clone()
            self._dist.all_reduce(full, group=self.group)
            out.copy_(full.chunk(self.world, dim=dim)[self.rank])
        return out

    def all_to_all(self, t, split_dim, concat_dim):
        ins = [c.contiguous() for c in t.chunk(self.world, dim=split_dim)]
        outs = [torch.empty_like(ins[0]) for _ in range(self.world)]
        if t.is_cuda:
            self._dist.all_to_all(outs, ins, group=self.group)
        else:  # gloo: emulate with all_gather
            gathered = [torch.empty((self.world,) + tuple(ins[0].shape), dtype=t.dtype) for _ in range(self.world)]
            self._dist.all_gather(gathered, torch.stack(ins), group=self.group)
            outs = [gathered[r][self.rank] for r in range(self.world)]
        return torch.cat(outs, dim=concat_dim)

    def broadcast(self, t, src=0):
        self._dist.broadcast(t, src=self.ranks[src], group=self.group)
        return t

    def send(self, t, dst):
        self._dist.send(t.contiguous(), dst=self.ranks[dst], group=self.group)

    def recv(self, t, src):
        self._dist.recv(t, src=self.ranks[src], group=self.group)
        return t

    def isend(self, t, dst):
        """Non-blocking send; returns a handle with ``wait()``. ``t`` must stay alive until then. With
        NCCL the transfer runs on the communicator's own stream behind the work that produced ``t``, so
        kernels launched afterwards on the current stream overlap it."""
        return self._dist.isend(t, dst=self.ranks[dst], group=self.group)

    def irecv(self, t, src):
        """Non-blocking receive into ``t``; ``wait()`` on the handle before reading it."""
        return self._dist.irecv(t, src=self.ranks[src], group=self.group)

    def barrier(self):
        self._dist.barrier(group=self.group)

    def all_gather_object(self, obj):
        out = [None] * self.world
        self._dist.all_gather_object(out, obj, group=self.group)
        return out

    def subgroup(self, ranks: Sequence[int]) -> "TorchDistComm":
        """Every rank of the parent must call this with the same ``ranks`` lists, in the same order.
        Returns the communicator on the member ranks and None on the others."""
        members = [self.ranks[r] for r in ranks]
        g = self._dist.new_group(members)
        if self.global_rank not in members:
            return None
        return TorchDistComm(g, members)


def init_comm(backend: Optional[str] = None, timeout_s: float = 600.0) -> Comm:
    """Create the world communicator from the torchrun environment (RANK / WORLD_SIZE /
    LOCAL_RANK / MASTER_ADDR / MASTER_PORT). Falls back to a single-rank communicator when the
    environment describes one process."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        log.decision("Collective", "transport=single ranks=1")
        return SingleComm()
    import torch.distributed as dist
    if not dist.is_initialized():
        use_cuda = torch.cuda.is_available()
        backend = backend or ("nccl" if use_cuda else "gloo")
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    comm = TorchDistComm()
    log.decision("Collective", f"transport={comm.transport} ranks={comm.world}")
    return comm
