"""Failure handling around the engine: retry with exponential back-off and jitter, a circuit
breaker (closed → open → half-open), bulkhead pools per request class, health checking,
cooperative shutdown, request time-outs, token-rate limiting, resource accounting and a
priority request queue.  All host-side, injectable clocks, no GPU state.
Reference parity: src/gpu/resilience.rs (``RetryPolicy``, ``CircuitBreaker``, ``BulkheadManager``),
``HealthChecker`` / ``ShutdownCoordinator`` / ``TimeoutManager`` / ``PriorityRequestQueue`` /
``TokenRateLimiter`` / ``ResourceTracker`` re-exported from src/gpu/mod.rs:41-125."""
from __future__ import annotations

import heapq
import itertools
import random
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple


class ErrorCategory(Enum):
    TRANSIENT = "transient"      # retry
    PERMANENT = "permanent"      # fail fast
    OVERLOAD = "overload"        # back off longer


def categorize(exc: BaseException) -> ErrorCategory:
    if isinstance(exc, (TimeoutError, ConnectionError, InterruptedError)):
        return ErrorCategory.TRANSIENT
    if isinstance(exc, (MemoryError, BlockingIOError)) or "queue is full" in str(exc).lower() or "out of memory" in str(exc).lower():
        return ErrorCategory.OVERLOAD
    return ErrorCategory.PERMANENT


@dataclass
class RetryConfig:
    max_retries: int = 3
    base_delay_s: float = 0.1
    max_delay_s: float = 30.0
    jitter: float = 0.1
    overload_factor: float = 4.0


class RetryPolicy:
    def __init__(self, cfg: Optional[RetryConfig] = None, rng: Optional[random.Random] = None):
        self.cfg, self.rng = cfg or RetryConfig(), rng or random.Random(0)

    def delay(self, attempt: int, category: ErrorCategory = ErrorCategory.TRANSIENT) -> float:
        d = self.cfg.base_delay_s * (2 ** attempt) * (self.cfg.overload_factor if category == ErrorCategory.OVERLOAD else 1.0)
        d = min(d, self.cfg.max_delay_s)
        return max(0.0, d * (1 + self.cfg.jitter * (2 * self.rng.random() - 1)))

    def should_retry(self, attempt: int, exc: BaseException) -> bool:
        return attempt < self.cfg.max_retries and categorize(exc) != ErrorCategory.PERMANENT

    def run(self, fn: Callable[[], Any], sleep: Callable[[float], None] = time.sleep) -> Any:
        attempt = 0
        while True:
            try:
                return fn()
            except Exception as e:
                if not self.should_retry(attempt, e):
                    raise
                sleep(self.delay(attempt, categorize(e)))
                attempt += 1


class CircuitState(Enum):
    CLOSED = "closed"
    OPEN = "open"
    HALF_OPEN = "half_open"


class CircuitOpen(RuntimeError):
    pass


class CircuitBreaker:
    def __init__(self, failure_threshold: int = 5, success_threshold: int = 2, timeout_s: float = 30.0, clock: Callable[[], float] = time.monotonic):
        self.failure_threshold, self.success_threshold, self.timeout_s, self.clock = failure_threshold, success_threshold, timeout_s, clock
        self.state, self.failures, self.successes, self.opened_at = CircuitState.CLOSED, 0, 0, 0.0
        self._lock = threading.Lock()

    def allow_request(self) -> bool:
        with self._lock:
            if self.state == CircuitState.OPEN and self.clock() - self.opened_at >= self.timeout_s:
                self.state, self.successes = CircuitState.HALF_OPEN, 0
            return self.state != CircuitState.OPEN

    def record_success(self) -> None:
        with self._lock:
            if self.state == CircuitState.HALF_OPEN:
                self.successes += 1
                if self.successes >= self.success_threshold:
                    self.state, self.failures = CircuitState.CLOSED, 0
            else:
                self.failures = 0

    def record_failure(self) -> None:
        with self._lock:
            self.failures += 1
            if self.state == CircuitState.HALF_OPEN or self.failures >= self.failure_threshold:
                self.state, self.opened_at = CircuitState.OPEN, self.clock()

    def call(self, fn: Callable[[], Any]) -> Any:
        if not self.allow_request():
            raise CircuitOpen("circuit is open")
        try:
            r = fn()
        except Exception:
            self.record_failure()
            raise
        self.record_success()
        return r


class BulkheadFull(RuntimeError):
    pass


class Bulkhead:
    """Separate concurrency pools per request class so that one class cannot starve the others."""

    def __init__(self, pools: Optional[Dict[str, int]] = None):
        self.limits = dict(pools or {"inference": 8, "embedding": 4, "batch": 2})
        self.in_use = {k: 0 for k in self.limits}
        self._lock = threading.Lock()

    def try_acquire(self, pool: str) -> bool:
        with self._lock:
            if self.in_use[pool] >= self.limits[pool]:
                return False
            self.in_use[pool] += 1
            return True

    def release(self, pool: str) -> None:
        with self._lock:
            self.in_use[pool] = max(0, self.in_use[pool] - 1)

    def run(self, pool: str, fn: Callable[[], Any]) -> Any:
        if not self.try_acquire(pool):
            raise BulkheadFull(f"bulkhead '{pool}' is full")
        try:
            return fn()
        finally:
            self.release(pool)

    def available(self, pool: str) -> int:
        return self.limits[pool] - self.in_use[pool]


class HealthChecker:
    def __init__(self):
        self.checks: Dict[str, Callable[[], bool]] = {}
        self.last: Dict[str, bool] = {}

    def register(self, name: str, check: Callable[[], bool]) -> None:
        self.checks[name] = check

    def check_all(self) -> Dict[str, bool]:
        for k, c in self.checks.items():
            try:
                self.last[k] = bool(c())
            except Exception:
                self.last[k] = False
        return dict(self.last)

    @property
    def healthy(self) -> bool:
        return all(self.check_all().values())


class ShutdownCoordinator:
    def __init__(self):
        self._ev = threading.Event()
        self.pending = 0
        self.handlers: List[Callable[[], None]] = []
        self._lock = threading.Lock()

    def register_handler(self, fn: Callable[[], None]) -> None:
        self.handlers.append(fn)

    def request_started(self) -> bool:
        with self._lock:
            if self._ev.is_set():
                return False
            self.pending += 1
            return True

    def request_completed(self) -> None:
        with self._lock:
            self.pending = max(0, self.pending - 1)

    @property
    def shutting_down(self) -> bool:
        return self._ev.is_set()

    def initiate(self, drain_timeout_s: float = 5.0, sleep=time.sleep) -> bool:
        self._ev.set()
        waited = 0.0
        while self.pending > 0 and waited < drain_timeout_s:
            sleep(0.01)
            waited += 0.01
        for h in self.handlers:
            h()
        return self.pending == 0


class TimeoutManager:
    def __init__(self, clock: Callable[[], float] = time.monotonic):
        self.clock = clock
        self.deadlines: Dict[Any, float] = {}

    def register(self, key, timeout_s: float) -> None:
        self.deadlines[key] = self.clock() + timeout_s

    def remove(self, key) -> None:
        self.deadlines.pop(key, None)

    def expired(self) -> List[Any]:
        now = self.clock()
        out = [k for k, d in self.deadlines.items() if d <= now]
        for k in out:
            del self.deadlines[k]
        return out


class TokenRateLimiter:
    """Token bucket (tokens = generated tokens, not requests)."""

    def __init__(self, rate_per_s: float, burst: float, clock: Callable[[], float] = time.monotonic):
        self.rate, self.burst, self.clock = rate_per_s, burst, clock
        self.level, self.t = burst, clock()

    def try_acquire(self, n: float = 1.0) -> bool:
        now = self.clock()
        self.level = min(self.burst, self.level + (now - self.t) * self.rate)
        self.t = now
        if self.level >= n:
            self.level -= n
            return True
        return False


class ResourceTracker:
    def __init__(self, memory_limit_bytes: int, compute_slots: int):
        self.memory_limit, self.compute_slots = memory_limit_bytes, compute_slots
        self.allocs: Dict[int, Tuple[int, int]] = {}
        self._ids = itertools.count(1)

    @property
    def memory_used(self) -> int:
        return sum(m for m, _ in self.allocs.values())

    @property
    def compute_used(self) -> int:
        return sum(c for _, c in self.allocs.values())

    def can_allocate(self, mem: int, compute: int = 1) -> bool:
        return self.memory_used + mem <= self.memory_limit and self.compute_used + compute <= self.compute_slots

    def allocate(self, mem: int, compute: int = 1) -> Optional[int]:
        if not self.can_allocate(mem, compute):
            return None
        i = next(self._ids)
        self.allocs[i] = (mem, compute)
        return i

    def release(self, alloc_id: int) -> None:
        self.allocs.pop(alloc_id, None)

    def usage(self) -> Tuple[float, float]:
        return self.memory_used / self.memory_limit if self.memory_limit else 0.0, self.compute_used / self.compute_slots if self.compute_slots else 0.0


class PriorityRequestQueue:
    """Highest priority first, FIFO within a priority."""

    def __init__(self):
        self._h: List[tuple] = []
        self._n = itertools.count()

    def push(self, item, priority: int = 0) -> None:
        heapq.heappush(self._h, (-priority, next(self._n), item))

    def pop(self):
        return heapq.heappop(self._h)[2] if self._h else None

    def __len__(self) -> int:
        return len(self._h)
