"""Benchmark harness pieces: CV-based stopping, thermal guard, inter-token-latency metrics,
result files, comparison / regression detection, and the convoy and saturation serving tests.
Reference parity: ``DynamicSampler`` / ``ThermalGuard`` / ``ItlMetrics`` (src/bench/mod.rs:68-414),
``bench-compare`` / ``bench-regression`` / convoy / saturation (src/cli/benchmark.rs:145-355)."""
from __future__ import annotations

import json
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from .stats import analyze_with_auto_select, summarize


@dataclass
class DynamicSampler:
    """Keep sampling until the coefficient of variation of the last ``window`` samples is below
    ``cv_threshold`` (stable) or ``max_samples`` is reached."""
    min_samples: int = 10
    max_samples: int = 1000
    cv_threshold: float = 0.05
    window: int = 20
    samples: List[float] = field(default_factory=list)

    def should_continue(self) -> bool:
        n = len(self.samples)
        if n < self.min_samples:
            return True
        if n >= self.max_samples:
            return False
        return self.current_cv() > self.cv_threshold

    def current_cv(self) -> float:
        w = np.asarray(self.samples[-self.window:], np.float64)
        return float(w.std(ddof=1) / w.mean()) if w.size > 1 and w.mean() else float("inf")

    def run(self, fn: Callable[[], float]) -> List[float]:
        while self.should_continue():
            self.samples.append(float(fn()))
        return self.samples


@dataclass
class ThermalGuard:
    """Pauses a benchmark while the device is hotter than ``max_temp_c`` and flags runs whose
    temperature moved by more than ``max_variance_c``.  The reader is injected (NVML on a GPU box)."""
    max_temp_c: float = 80.0
    cooldown_threshold_c: float = 70.0
    cooldown_sleep_s: float = 1.0
    max_variance_c: float = 10.0
    temps: List[float] = field(default_factory=list)

    def record(self, t: float) -> None:
        self.temps.append(float(t))

    def needs_cooldown(self, t: float) -> bool:
        return t > self.max_temp_c

    def cooldown(self, read_temp: Callable[[], float], sleep=time.sleep, max_wait_s: float = 60.0) -> float:
        waited = 0.0
        while read_temp() > self.cooldown_threshold_c and waited < max_wait_s:
            sleep(self.cooldown_sleep_s)
            waited += self.cooldown_sleep_s
        return waited

    def is_valid_run(self) -> bool:
        return not self.temps or (max(self.temps) - min(self.temps)) <= self.max_variance_c


def nvml_temperature_reader(index: int = 0) -> Callable[[], float]:
    import pynvml
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(index)
    return lambda: float(pynvml.nvmlDeviceGetTemperature(h, pynvml.NVML_TEMPERATURE_GPU))


@dataclass
class ItlMetrics:
    median_ms: float
    p99_ms: float
    p999_ms: float
    std_ms: float
    jitter_cv: float

    @classmethod
    def from_timestamps(cls, token_times: Sequence[float]) -> "ItlMetrics":
        d = np.diff(np.asarray(token_times, np.float64)) * 1e3
        if d.size == 0:
            return cls(0, 0, 0, 0, 0)
        return cls(float(np.median(d)), float(np.percentile(d, 99)), float(np.percentile(d, 99.9)), float(d.std()), float(d.std() / d.mean()) if d.mean() else 0.0)


@dataclass
class BenchResult:
    name: str
    unit: str
    samples: List[float]
    higher_is_better: bool = False
    meta: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return {**asdict(self), "summary": asdict(summarize(self.samples))}


def save_results(path: str, results: Sequence[BenchResult]) -> None:
    with open(path, "w") as f:
        json.dump({"version": 1, "results": [r.to_json() for r in results]}, f, indent=1)


def load_results(path: str) -> Dict[str, BenchResult]:
    with open(path) as f:
        d = json.load(f)
    return {r["name"]: BenchResult(r["name"], r["unit"], r["samples"], r.get("higher_is_better", False), r.get("meta", {})) for r in d["results"]}


@dataclass
class Comparison:
    name: str
    baseline: float
    current: float
    change_pct: float          # positive = better
    p_value: float
    verdict: str               # "improved" | "regressed" | "unchanged"


def compare_results(base: Dict[str, BenchResult], cur: Dict[str, BenchResult], threshold_pct: float = 5.0, alpha: float = 0.05) -> List[Comparison]:
    out = []
    for name, b in base.items():
        c = cur.get(name)
        if c is None:
            continue
        mb, mc = float(np.mean(b.samples)), float(np.mean(c.samples))
        change = (mc - mb) / mb * 100 if mb else 0.0
        if not b.higher_is_better:
            change = -change
        p = analyze_with_auto_select(b.samples, c.samples, alpha).p_value if min(len(b.samples), len(c.samples)) >= 3 else 0.0
        sig = p < alpha and abs(change) >= threshold_pct
        out.append(Comparison(name, mb, mc, change, p, ("improved" if change > 0 else "regressed") if sig else "unchanged"))
    return out


def has_regression(cmp: Sequence[Comparison]) -> bool:
    return any(c.verdict == "regressed" for c in cmp)


# -- serving stress tests --------------------------------------------------------------------------
def convoy_test(serving, n_long: int = 2, n_short: int = 8, long_tokens: int = 64, short_tokens: int = 4, prompt_len: int = 8, vocab: int = 100,
                timeout: float = 60.0) -> dict:
    """Long requests first, then short ones: with continuous batching the short ones must not wait
    for the long ones to drain (head-of-line blocking check)."""
    from ..runtime.scheduler import Request
    done: Dict[int, float] = {}
    ev = threading.Event()
    total = n_long + n_short
    t0 = time.monotonic()

    def fin(kind, i):
        def _f(_r):
            done[(kind, i)] = time.monotonic() - t0
            if len(done) == total:
                ev.set()
        return _f
    rng = np.random.default_rng(0)
    for i in range(n_long):
        serving.submit(Request(list(rng.integers(1, vocab, prompt_len)), max_tokens=long_tokens, on_finish=fin("long", i)))
    for i in range(n_short):
        serving.submit(Request(list(rng.integers(1, vocab, prompt_len)), max_tokens=short_tokens, on_finish=fin("short", i)))
    ok = ev.wait(timeout)
    longs = [v for (k, _), v in done.items() if k == "long"]
    shorts = [v for (k, _), v in done.items() if k == "short"]
    return {"completed": len(done), "total": total, "ok": ok, "short_p50_s": float(np.median(shorts)) if shorts else None,
            "long_p50_s": float(np.median(longs)) if longs else None,
            "hol_blocking": bool(shorts and longs and np.median(shorts) >= min(longs))}


def saturation_test(serving, concurrency: int = 16, requests: int = 64, max_tokens: int = 8, prompt_len: int = 8, vocab: int = 100, timeout: float = 120.0) -> dict:
    """Closed-loop load: ``concurrency`` clients each issue requests back to back."""
    from ..runtime.scheduler import QueueFull
    lat: List[float] = []
    rejected = [0]
    lock = threading.Lock()
    counter = iter(range(requests))
    rng = np.random.default_rng(1)
    prompts = [list(map(int, rng.integers(1, vocab, prompt_len))) for _ in range(requests)]

    def client():
        while True:
            with lock:
                i = next(counter, None)
            if i is None:
                return
            t = time.monotonic()
            try:
                serving.generate(prompts[i], timeout=timeout, max_tokens=max_tokens)
                with lock:
                    lat.append(time.monotonic() - t)
            except QueueFull:
                with lock:
                    rejected[0] += 1
    t0 = time.monotonic()
    th = [threading.Thread(target=client) for _ in range(concurrency)]
    [t.start() for t in th]
    [t.join(timeout) for t in th]
    wall = time.monotonic() - t0
    s = summarize([1e3 * x for x in lat])
    return {"completed": len(lat), "rejected": rejected[0], "wall_s": wall, "req_per_s": len(lat) / wall if wall else 0.0,
            "tok_per_s": len(lat) * max_tokens / wall if wall else 0.0, "latency_ms": asdict(s)}
