"""Process metrics (Prometheus text format).

Keeps the reference's two metric names (``hartsyinference_requests_total``,
``hartsyinference_queue_pending``; src/HartsyInference.API/Metrics.cs) and adds serving metrics.
Uses ``prometheus_client`` when it is installed, otherwise a small built-in registry with the same
exposition format.
"""
from __future__ import annotations

import threading
from collections import defaultdict


class _Registry:
    def __init__(self):
        self._lock = threading.Lock()
        self.counters: dict[tuple, float] = defaultdict(float)
        self.gauges: dict[tuple, float] = {}
        self.help: dict[str, tuple[str, str]] = {}

    def declare(self, name: str, kind: str, doc: str) -> None:
        self.help[name] = (kind, doc)

    def inc(self, name: str, value: float = 1.0, **labels) -> None:
        with self._lock:
            self.counters[(name, tuple(sorted(labels.items())))] += value

    def set(self, name: str, value: float, **labels) -> None:
        with self._lock:
            self.gauges[(name, tuple(sorted(labels.items())))] = value

    def get(self, name: str, **labels) -> float:
        key = (name, tuple(sorted(labels.items())))
        with self._lock:
            return self.counters.get(key, self.gauges.get(key, 0.0))

    def render(self) -> str:
        lines = []
        with self._lock:
            items = list(self.counters.items()) + list(self.gauges.items())
        seen = set()
        for (name, labels), v in sorted(items):
            if name not in seen:
                kind, doc = self.help.get(name, ("gauge", name))
                lines.append(f"# HELP {name} {doc}")
                lines.append(f"# TYPE {name} {kind}")
                seen.add(name)
            lab = ",".join(f'{k}="{val}"' for k, val in labels)
            lines.append(f"{name}{{{lab}}} {v}" if lab else f"{name} {v}")
        return "\n".join(lines) + "\n"


REGISTRY = _Registry()
for _n, _k, _d in (
    ("hartsyinference_requests_total", "counter", "requests by route and outcome"),
    ("hartsyinference_queue_pending", "gauge", "requests waiting or running"),
    ("hartsyinference_tokens_total", "counter", "generated tokens"),
    ("hartsyinference_ttft_seconds", "gauge", "time to first token of the last request"),
    ("hartsyinference_decode_tok_s", "gauge", "decode throughput of the last request"),
    ("hartsyinference_kv_pages_used", "gauge", "KV pages in use"),
    ("hartsyinference_batch_size", "gauge", "sequences in the last decode batch"),
    ("hartsyinference_step_seconds", "gauge", "duration of the last denoise step by model"),
):
    REGISTRY.declare(_n, _k, _d)
