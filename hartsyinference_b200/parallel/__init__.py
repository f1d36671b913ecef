"""Parallel execution: process groups, the NVLink symmetric heap, fused compute+collective
kernels, and the TP / SP / EP / CFG / PP plans."""
from .comm import Comm, SingleComm, TorchDistComm, init_comm  # noqa: F401
from .config import ParallelConfig  # noqa: F401
