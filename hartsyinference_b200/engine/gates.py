"""Device gates and the bounded inference queue.

``DeviceGate`` holds one lock per device ordinal; a request that needs several devices acquires
them in ascending order, which cannot deadlock (the reference's DeviceGate does the same with
SemaphoreSlim, src/HartsyInference.Engine/DeviceGate.cs; ``HARTSY_SAME_GPU_CONCURRENT`` maps to the
``same_gpu_concurrent`` flag). ``InferenceQueue`` bounds the number of waiting requests and raises
``QueueFullError`` (HTTP 429) beyond it (src/HartsyInference.Engine/InferenceQueue.cs).
"""
from __future__ import annotations

import contextlib
import threading
from typing import Iterable

from .. import config
from ..exceptions import QueueFullError


class DeviceGate:
    def __init__(self):
        self._locks: dict[int, threading.Semaphore] = {}
        self._meta = threading.Lock()

    def _lock(self, ordinal: int) -> threading.Semaphore:
        with self._meta:
            if ordinal not in self._locks:
                self._locks[ordinal] = threading.Semaphore(2 if config.get("same_gpu_concurrent") else 1)
            return self._locks[ordinal]

    @contextlib.contextmanager
    def acquire(self, ordinals: Iterable[int]):
        order = sorted(set(ordinals))
        held = []
        try:
            for o in order:
                lk = self._lock(o)
                lk.acquire()
                held.append(lk)
            yield
        finally:
            for lk in reversed(held):
                lk.release()

    def acquire_all(self, count: int):
        return self.acquire(range(count))


class InferenceQueue:
    """Counting gate: at most ``max_concurrency`` running, at most ``max_depth`` waiting."""

    def __init__(self, max_concurrency: int = 1, max_depth: int = 16):
        self.max_concurrency, self.max_depth = max_concurrency, max_depth
        self._running = 0
        self._waiting = 0
        self._cv = threading.Condition()

    @property
    def pending(self) -> int:
        with self._cv:
            return self._waiting + self._running

    @contextlib.contextmanager
    def slot(self):
        with self._cv:
            if self._running >= self.max_concurrency and self._waiting >= self.max_depth:
                raise QueueFullError(f"queue full ({self._waiting} waiting, depth {self.max_depth})")
            self._waiting += 1
            try:
                while self._running >= self.max_concurrency:
                    self._cv.wait()
            finally:
                self._waiting -= 1
            self._running += 1
        try:
            yield
        finally:
            with self._cv:
                self._running -= 1
                self._cv.notify()
