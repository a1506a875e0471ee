"""Serving metrics: request / token counters with Prometheus text exposition, latency histograms
with percentiles (TTFT, inter-token latency, end-to-end), and CPU-vs-GPU dispatch accounting.

Metric names follow the reference (``realizar_requests_total`` ... ``realizar_uptime_seconds``,
src/metrics.rs:21-160; dispatch metrics src/gguf/inference_types.rs:418, src/gguf/latency.rs:8-140;
latency histogram src/observability/mod.rs:47-421), extended with TTFT / ITL / queue / KV gauges.
"""
from __future__ import annotations

import bisect
import threading
import time
from typing import Dict, List, Optional, Sequence


class LatencyHistogram:
    """Fixed-bucket histogram (seconds) that also keeps a bounded reservoir for exact percentiles."""
    DEFAULT_BUCKETS = (0.001, 0.0025, 0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0)

    def __init__(self, buckets: Sequence[float] = DEFAULT_BUCKETS, reservoir: int = 4096):
        self.buckets = tuple(buckets)
        self.counts = [0] * (len(self.buckets) + 1)
        self.total, self.sum = 0, 0.0
        self._res: List[float] = []
        self._cap = reservoir
        self._lock = threading.Lock()

    def observe(self, seconds: float) -> None:
        with self._lock:
            self.counts[bisect.bisect_left(self.buckets, seconds)] += 1
            self.total += 1
            self.sum += seconds
            if len(self._res) < self._cap:
                self._res.append(seconds)
            else:
                self._res[self.total % self._cap] = seconds

    def percentile(self, p: float) -> float:
        with self._lock:
            if not self._res:
                return 0.0
            s = sorted(self._res)
        return s[min(len(s) - 1, int(round(p / 100.0 * (len(s) - 1))))]

    @property
    def mean(self) -> float:
        return self.sum / self.total if self.total else 0.0

    def variance(self) -> float:
        with self._lock:
            if len(self._res) < 2:
                return 0.0
            m = sum(self._res) / len(self._res)
            return sum((x - m) ** 2 for x in self._res) / (len(self._res) - 1)

    def prometheus(self, name: str, help_: str) -> str:
        out = [f"# HELP {name} {help_}", f"# TYPE {name} histogram"]
        cum = 0
        for b, c in zip(self.buckets, self.counts):
            cum += c
            out.append(f'{name}_bucket{{le="{b}"}} {cum}')
        out.append(f'{name}_bucket{{le="+Inf"}} {self.total}')
        out.append(f"{name}_sum {self.sum}")
        out.append(f"{name}_count {self.total}")
        return "\n".join(out)


class MetricsCollector:
    def __init__(self):
        self._lock = threading.Lock()
        self.start = time.time()
        self.requests_total = self.requests_successful = self.requests_failed = 0
        self.tokens_generated = 0
        self.inference_time = 0.0
        self.ttft = LatencyHistogram()
        self.itl = LatencyHistogram()
        self.e2e = LatencyHistogram()
        self.gauges: Dict[str, float] = {}

    def record_success(self, tokens: int, seconds: float, ttft: Optional[float] = None, token_times: Optional[Sequence[float]] = None) -> None:
        with self._lock:
            self.requests_total += 1
            self.requests_successful += 1
            self.tokens_generated += tokens
            self.inference_time += seconds
        self.e2e.observe(seconds)
        if ttft is not None:
            self.ttft.observe(ttft)
        if token_times:
            for a, b in zip(token_times, token_times[1:]):
                self.itl.observe(b - a)

    def record_failure(self) -> None:
        with self._lock:
            self.requests_total += 1
            self.requests_failed += 1

    def set_gauge(self, name: str, value: float) -> None:
        self.gauges[name] = float(value)

    def snapshot(self) -> dict:
        up = max(1e-9, time.time() - self.start)
        with self._lock:
            rt, rs, rf, tg, it = self.requests_total, self.requests_successful, self.requests_failed, self.tokens_generated, self.inference_time
        return {"requests_total": rt, "requests_successful": rs, "requests_failed": rf, "tokens_generated": tg,
                "inference_time_seconds": it, "requests_per_second": rt / up, "tokens_per_second": tg / it if it > 0 else 0.0,
                "avg_latency_ms": 1e3 * it / rs if rs else 0.0, "error_rate": rf / rt if rt else 0.0, "uptime_seconds": up,
                "ttft_p50_ms": 1e3 * self.ttft.percentile(50), "ttft_p99_ms": 1e3 * self.ttft.percentile(99),
                "itl_p50_ms": 1e3 * self.itl.percentile(50), "itl_p99_ms": 1e3 * self.itl.percentile(99), **self.gauges}

    def prometheus(self) -> str:
        s = self.snapshot()
        lines = []
        for key, typ, help_ in (("requests_total", "counter", "Total requests"), ("requests_successful", "counter", "Successful requests"),
                                ("requests_failed", "counter", "Failed requests"), ("tokens_generated", "counter", "Tokens generated"),
                                ("inference_time_seconds", "counter", "Time spent generating"), ("requests_per_second", "gauge", "Request rate"),
                                ("tokens_per_second", "gauge", "Generation throughput"), ("avg_latency_ms", "gauge", "Mean request latency"),
                                ("error_rate", "gauge", "Failed / total"), ("uptime_seconds", "gauge", "Process uptime")):
            lines += [f"# HELP realizar_{key} {help_}", f"# TYPE realizar_{key} {typ}", f"realizar_{key} {s[key]}"]
        for g, v in self.gauges.items():
            lines += [f"# TYPE realizar_{g} gauge", f"realizar_{g} {v}"]
        lines.append(self.ttft.prometheus("realizar_ttft_seconds", "Time to first token"))
        lines.append(self.itl.prometheus("realizar_itl_seconds", "Inter-token latency"))
        lines.append(self.e2e.prometheus("realizar_request_seconds", "End-to-end request latency"))
        return "\n".join(lines) + "\n"


class DispatchMetrics:
    """Counts and latencies of work dispatched to the CPU path vs the GPU path."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.cpu, self.gpu = 0, 0
        self.cpu_lat, self.gpu_lat = LatencyHistogram(), LatencyHistogram()
        self.start = time.time()

    def record(self, backend: str, seconds: float) -> None:
        if backend == "gpu":
            self.gpu += 1
            self.gpu_lat.observe(seconds)
        else:
            self.cpu += 1
            self.cpu_lat.observe(seconds)

    def to_dict(self) -> dict:
        tot = self.cpu + self.gpu
        def lat(h):
            return {"count": h.total, "mean_us": 1e6 * h.mean, "p50_us": 1e6 * h.percentile(50), "p95_us": 1e6 * h.percentile(95),
                    "p99_us": 1e6 * h.percentile(99), "variance": h.variance()}
        return {"cpu_dispatches": self.cpu, "gpu_dispatches": self.gpu, "total_dispatches": tot,
                "gpu_dispatch_ratio": self.gpu / tot if tot else 0.0, "cpu_latency": lat(self.cpu_lat), "gpu_latency": lat(self.gpu_lat),
                "elapsed_seconds": time.time() - self.start}

    def prometheus(self) -> str:
        d = self.to_dict()
        return (f"# TYPE realizar_dispatch_cpu_total counter\nrealizar_dispatch_cpu_total {d['cpu_dispatches']}\n"
                f"# TYPE realizar_dispatch_gpu_total counter\nrealizar_dispatch_gpu_total {d['gpu_dispatches']}\n"
                f"# TYPE realizar_dispatch_gpu_ratio gauge\nrealizar_dispatch_gpu_ratio {d['gpu_dispatch_ratio']}\n")
