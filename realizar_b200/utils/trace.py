"""Tracing: the inference state machine that emits step events (TOKENIZE, EMBED,
TRANSFORMER_BLOCK, LM_HEAD, SAMPLE, DECODE) in the ``TaskStateEntered`` / ``TaskStateExited``
JSON form, tensor statistics for divergence hunting, a CPU-vs-GPU layer diff, and a brick-level
timer with device events.

Reference parity: ``InferenceTracer`` (src/inference_trace/mod.rs:30-448), ``BrickTracer`` /
``TraceDiff`` (src/brick/tracer.rs:53-339), ``BrickProfiler`` (src/brick/profiler.rs:47-165),
``ForwardTrace`` / ``ActivationStats`` (src/apr_transformer/mod.rs:179-341).
"""
from __future__ import annotations

import json
import os
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import numpy as np

STEPS = ("LOAD", "TOKENIZE", "EMBED", "TRANSFORMER_BLOCK", "LM_HEAD", "SAMPLE", "DECODE")


@dataclass
class TensorStats:
    mean: float
    std: float
    l2: float
    min: float
    max: float
    nan_count: int
    inf_count: int
    size: int

    @classmethod
    def of(cls, x) -> "TensorStats":
        a = np.asarray(x.detach().float().cpu().numpy() if hasattr(x, "detach") else x, dtype=np.float64).ravel()
        fin = a[np.isfinite(a)]
        if fin.size == 0:
            return cls(0.0, 0.0, 0.0, 0.0, 0.0, int(np.isnan(a).sum()), int(np.isinf(a).sum()), int(a.size))
        return cls(float(fin.mean()), float(fin.std()), float(np.linalg.norm(fin)), float(fin.min()), float(fin.max()),
                   int(np.isnan(a).sum()), int(np.isinf(a).sum()), int(a.size))

    @property
    def healthy(self) -> bool:
        return self.nan_count == 0 and self.inf_count == 0


class InferenceTracer:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.events: List[dict] = []
        self._open: Dict[str, float] = {}
        self._id = 0

    def _emit(self, kind: str, name: str, details: dict) -> None:
        if not self.enabled:
            return
        self._id += 1
        self.events.append({"id": self._id, "type": kind, "timestamp": time.time(), "details": {"name": name, **details}})

    def enter(self, step: str, **inputs) -> None:
        self._open[step] = time.perf_counter()
        self._emit("TaskStateEntered", step, {"input": inputs})

    def exit(self, step: str, **outputs) -> None:
        t0 = self._open.pop(step, None)
        dur = 1e3 * (time.perf_counter() - t0) if t0 is not None else None
        self._emit("TaskStateExited", step, {"output": outputs, "duration_ms": dur})

    def tensor(self, step: str, name: str, x) -> None:
        if self.enabled:
            self._emit("TensorStats", step, {"tensor": name, **asdict(TensorStats.of(x))})

    def to_json(self) -> str:
        return json.dumps({"events": self.events}, indent=1)

    def write(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_json())

    def summary(self) -> Dict[str, float]:
        return {e["details"]["name"]: e["details"]["duration_ms"] for e in self.events if e["type"] == "TaskStateExited" and e["details"]["duration_ms"] is not None}


@dataclass
class TraceDiff:
    name: str
    cosine: float
    max_abs: float
    rel_l2: float

    @property
    def ok(self) -> bool:
        return self.cosine >= 0.99


def compare_traces(a: Dict[str, np.ndarray], b: Dict[str, np.ndarray]) -> List[TraceDiff]:
    """Per-stage diff of two activation dictionaries (e.g. oracle vs GPU); stops being meaningful after the first bad stage."""
    out = []
    for k in a:
        if k not in b:
            continue
        x, y = np.asarray(a[k], np.float64).ravel(), np.asarray(b[k], np.float64).ravel()
        n = min(x.size, y.size)
        x, y = x[:n], y[:n]
        den = np.linalg.norm(x) * np.linalg.norm(y)
        out.append(TraceDiff(k, float(x @ y / den) if den > 0 else 1.0, float(np.abs(x - y).max()) if n else 0.0,
                             float(np.linalg.norm(x - y) / max(1e-30, np.linalg.norm(x)))))
    return out


def first_divergence(diffs: List[TraceDiff]) -> Optional[TraceDiff]:
    return next((d for d in diffs if not d.ok), None)


@contextmanager
def nvtx_range(name: str):
    """An NVTX range around a piece of host code that launches GPU work, when ``RLZ_NVTX=1`` and a CUDA device is present
    (timeline tools group the launches under it); otherwise nothing."""
    on = os.environ.get("RLZ_NVTX", "0") != "0"
    if on:
        import torch
        on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class BrickProfiler:
    """Accumulates per-brick timings.  On a CUDA device the bricks are bracketed with events on the
    current stream and resolved at ``summary()`` (no synchronisation inside the hot loop); with ``RLZ_NVTX=1`` every brick is
    also an NVTX range."""

    def __init__(self, cuda: Optional[bool] = None):
        import torch
        self.cuda = torch.cuda.is_available() if cuda is None else cuda
        self.totals: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}
        self._pending: List[tuple] = []

    @contextmanager
    def brick(self, name: str):
        if self.cuda:
            import torch
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            with nvtx_range(name):
                yield
            e1.record()
            self._pending.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            yield
            self._add(name, 1e3 * (time.perf_counter() - t0))

    def _add(self, name: str, ms: float) -> None:
        self.totals[name] = self.totals.get(name, 0.0) + ms
        self.counts[name] = self.counts.get(name, 0) + 1

    def summary(self) -> Dict[str, dict]:
        if self._pending:
            import torch
            torch.cuda.synchronize()
            for name, e0, e1 in self._pending:
                self._add(name, e0.elapsed_time(e1))
            self._pending = []
        tot = sum(self.totals.values()) or 1.0
        return {k: {"total_ms": v, "count": self.counts[k], "avg_us": 1e3 * v / self.counts[k], "share": v / tot}
                for k, v in sorted(self.totals.items(), key=lambda kv: -kv[1])}

    def bottleneck(self) -> Optional[str]:
        s = self.summary()
        return next(iter(s)) if s else None
