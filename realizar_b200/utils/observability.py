"""Observability primitives: W3C trace context propagation, spans, latency histograms with
percentile queries and Prometheus exposition, and deterministic A/B variant assignment.
Reference parity: ``TraceContext`` / ``LatencyHistogram`` / span structs / ``ABTest``
(src/observability/mod.rs:47-421)."""
from __future__ import annotations

import hashlib
import os
import time
from bisect import bisect_left
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class TraceContext:
    trace_id: str            # 32 hex
    span_id: str             # 16 hex
    sampled: bool = True
    parent_span_id: Optional[str] = None

    @classmethod
    def new(cls) -> "TraceContext":
        return cls(os.urandom(16).hex(), os.urandom(8).hex())

    @classmethod
    def from_traceparent(cls, header: str) -> Optional["TraceContext"]:
        """``00-<trace id>-<parent span id>-<flags>``; anything malformed yields None (a new trace is started)."""
        parts = header.strip().split("-")
        if len(parts) != 4 or parts[0] != "00" or len(parts[1]) != 32 or len(parts[2]) != 16 or len(parts[3]) != 2:
            return None
        try:
            int(parts[1], 16); int(parts[2], 16); flags = int(parts[3], 16)
        except ValueError:
            return None
        if parts[1] == "0" * 32 or parts[2] == "0" * 16:
            return None
        return cls(parts[1], os.urandom(8).hex(), bool(flags & 1), parts[2])

    def to_traceparent(self) -> str:
        return f"00-{self.trace_id}-{self.span_id}-{'01' if self.sampled else '00'}"

    def child(self) -> "TraceContext":
        return TraceContext(self.trace_id, os.urandom(8).hex(), self.sampled, self.span_id)


@dataclass
class Span:
    name: str
    context: TraceContext
    start_ns: int = field(default_factory=time.time_ns)
    end_ns: Optional[int] = None
    attributes: Dict[str, object] = field(default_factory=dict)
    status: str = "unset"

    def set(self, key: str, value) -> "Span":
        self.attributes[key] = value
        return self

    def end(self, ok: bool = True) -> "Span":
        self.end_ns, self.status = time.time_ns(), "ok" if ok else "error"
        return self

    @property
    def duration_ms(self) -> Optional[float]:
        return None if self.end_ns is None else (self.end_ns - self.start_ns) / 1e6

    def to_otel(self) -> dict:
        return {"traceId": self.context.trace_id, "spanId": self.context.span_id, "parentSpanId": self.context.parent_span_id, "name": self.name,
                "startTimeUnixNano": self.start_ns, "endTimeUnixNano": self.end_ns, "status": {"code": self.status},
                "attributes": [{"key": k, "value": v} for k, v in self.attributes.items()]}


class LatencyHistogram:
    DEFAULT_BOUNDS_MS = (0.5, 1, 2.5, 5, 10, 25, 50, 100, 250, 500, 1000, 2500, 5000, 10000)

    def __init__(self, bounds_ms: Sequence[float] = DEFAULT_BOUNDS_MS):
        self.bounds = list(bounds_ms)
        self.counts = [0] * (len(self.bounds) + 1)
        self.total, self.sum_ms = 0, 0.0

    def observe(self, ms: float) -> None:
        self.counts[bisect_left(self.bounds, ms)] += 1
        self.total += 1
        self.sum_ms += ms

    def percentile(self, q: float) -> float:
        """Upper bound of the bucket that holds the q-th percentile (inf for the overflow bucket)."""
        if self.total == 0:
            return 0.0
        target, cum = q / 100.0 * self.total, 0
        for i, c in enumerate(self.counts):
            cum += c
            if cum >= target:
                return self.bounds[i] if i < len(self.bounds) else float("inf")
        return float("inf")

    @property
    def mean_ms(self) -> float:
        return self.sum_ms / self.total if self.total else 0.0

    def to_prometheus(self, name: str) -> str:
        lines, cum = [f"# TYPE {name} histogram"], 0
        for b, c in zip(self.bounds, self.counts):
            cum += c
            lines.append(f'{name}_bucket{{le="{b / 1e3:g}"}} {cum}')
        lines += [f'{name}_bucket{{le="+Inf"}} {self.total}', f"{name}_sum {self.sum_ms / 1e3:g}", f"{name}_count {self.total}"]
        return "\n".join(lines) + "\n"


@dataclass
class ABTest:
    """Deterministic assignment of a key (user, request) to a weighted variant, with per-variant outcome counters."""
    name: str
    variants: Dict[str, float]
    outcomes: Dict[str, List[float]] = field(default_factory=dict)

    def assign(self, key: str) -> str:
        h = int.from_bytes(hashlib.sha256(f"{self.name}:{key}".encode()).digest()[:8], "big") / 2 ** 64
        tot, acc = sum(self.variants.values()), 0.0
        for v, w in self.variants.items():
            acc += w / tot
            if h < acc:
                return v
        return next(reversed(self.variants))

    def record(self, variant: str, value: float) -> None:
        self.outcomes.setdefault(variant, []).append(value)

    def summary(self) -> Dict[str, dict]:
        return {v: {"n": len(xs), "mean": sum(xs) / len(xs) if xs else 0.0} for v, xs in self.outcomes.items()}
