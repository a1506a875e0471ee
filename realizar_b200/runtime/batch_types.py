"""Small host-side value types used around the engine: token batches, a speculative token buffer,
an asynchronous result handle, a bounded asynchronous request queue, an event notifier, inference
counters, a micro-batch assembler and a multi-request scheduler with FCFS / SJF / round-robin
policies.  Reference parity: ``TokenBatch``, ``SpeculativeBuffer``, ``AsyncGpuResult``,
``AsyncRequestQueue``, ``InferenceEventNotifier``, ``InferenceMetrics``, ``InferenceBatchScheduler``
(re-exports in src/gpu/mod.rs:41-125), ``MicroBatch`` / ``BatchToken`` / ``SequenceBatch``
(src/scheduler/mod_num_slots_idle.rs:4-440), ``MultiRequestScheduler`` / ``BatchRequestCollector``
(src/gguf/batch_scheduler*.rs)."""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence


class TokenBatch:
    """Accumulates tokens until ``capacity`` is reached; ``push`` returns the full batch when it fills."""

    def __init__(self, capacity: int):
        self.capacity, self.tokens = capacity, []

    def push(self, token: int) -> Optional[List[int]]:
        self.tokens.append(int(token))
        return self.flush() if len(self.tokens) >= self.capacity else None

    def flush(self) -> List[int]:
        out, self.tokens = self.tokens, []
        return out

    def __len__(self) -> int:
        return len(self.tokens)


class SpeculativeBuffer:
    """Draft tokens with their confidences; ``verify`` keeps the prefix that matches the target."""

    def __init__(self, capacity: int = 8):
        self.capacity, self.items = capacity, []

    def add_candidate(self, token: int, confidence: float) -> bool:
        if len(self.items) >= self.capacity:
            return False
        self.items.append((int(token), float(confidence)))
        return True

    def verify(self, actual: Sequence[int]) -> tuple:
        n = 0
        for (t, _), a in zip(self.items, actual):
            if t != a:
                break
            n += 1
        return n, (None if n == len(self.items) else n)

    def accept(self, n: int) -> None:
        del self.items[:n]

    def reject(self) -> None:
        self.items.clear()

    def __len__(self) -> int:
        return len(self.items)


class AsyncGpuResult:
    """A result that becomes available later (set by the engine thread, awaited by the caller)."""

    def __init__(self):
        self._ev, self._val, self._err = threading.Event(), None, None

    def set_result(self, value) -> None:
        self._val = value
        self._ev.set()

    def set_error(self, err: BaseException) -> None:
        self._err = err
        self._ev.set()

    def is_ready(self) -> bool:
        return self._ev.is_set()

    def wait(self, timeout: Optional[float] = None):
        if not self._ev.wait(timeout):
            raise TimeoutError("result not ready")
        if self._err is not None:
            raise self._err
        return self._val


class AsyncRequestQueue:
    def __init__(self, capacity: int):
        self.capacity, self.q = capacity, deque()
        self._lock = threading.Lock()

    def try_push(self, item) -> bool:
        with self._lock:
            if len(self.q) >= self.capacity:
                return False
            self.q.append(item)
            return True

    def try_pop(self):
        with self._lock:
            return self.q.popleft() if self.q else None

    def __len__(self) -> int:
        return len(self.q)

    @property
    def is_full(self) -> bool:
        return len(self.q) >= self.capacity


class InferenceEventNotifier:
    def __init__(self):
        self.handlers: List[Callable[[int, float, int], None]] = []

    def register(self, fn: Callable[[int, float, int], None]) -> None:
        self.handlers.append(fn)

    def notify(self, request_id: int, latency_ms: float, tokens: int) -> None:
        for h in self.handlers:
            h(request_id, latency_ms, tokens)

    def clear(self) -> None:
        self.handlers.clear()


@dataclass
class InferenceMetrics:
    total_inferences: int = 0
    total_tokens: int = 0
    total_latency_ms: float = 0.0
    latencies_ms: List[float] = field(default_factory=list)
    started: float = field(default_factory=time.monotonic)

    def record(self, latency_ms: float, tokens: int) -> None:
        self.total_inferences += 1
        self.total_tokens += tokens
        self.total_latency_ms += latency_ms
        self.latencies_ms.append(latency_ms)

    def percentile(self, q: float) -> float:
        if not self.latencies_ms:
            return 0.0
        xs = sorted(self.latencies_ms)
        return xs[min(len(xs) - 1, int(q / 100.0 * len(xs)))]

    def throughput(self) -> float:
        dt = time.monotonic() - self.started
        return self.total_tokens / dt if dt > 0 else 0.0


@dataclass
class BatchToken:
    token: int
    seq_id: int
    position: int
    is_prompt: bool = False


@dataclass
class MicroBatch:
    """One engine iteration's worth of tokens: prompt chunks and decode tokens of several sequences."""
    tokens: List[BatchToken] = field(default_factory=list)
    max_tokens: int = 512

    def add(self, t: BatchToken) -> bool:
        if len(self.tokens) >= self.max_tokens:
            return False
        self.tokens.append(t)
        return True

    @property
    def num_prompt(self) -> int:
        return sum(1 for t in self.tokens if t.is_prompt)

    @property
    def num_decode(self) -> int:
        return len(self.tokens) - self.num_prompt

    def sequences(self) -> List[int]:
        return sorted({t.seq_id for t in self.tokens})


class SchedulingPolicy(Enum):
    FCFS = "fcfs"
    SJF = "sjf"           # shortest remaining job first
    ROUND_ROBIN = "rr"


class MultiRequestScheduler:
    """Chooses which pending request runs next under a policy (host-side; the continuous-batching
    loop in ``runtime.scheduler`` is what the server uses, this is the library form with pluggable policies)."""

    def __init__(self, policy: SchedulingPolicy = SchedulingPolicy.FCFS, max_concurrent: int = 4):
        self.policy, self.max_concurrent = policy, max_concurrent
        self.pending: Deque[dict] = deque()
        self.active: List[dict] = []
        self._next = 0
        self._rr = 0

    def submit(self, prompt_len: int, max_tokens: int) -> int:
        rid = self._next
        self._next += 1
        self.pending.append({"id": rid, "remaining": max_tokens, "prompt_len": prompt_len, "submitted": time.monotonic()})
        return rid

    def admit(self) -> List[int]:
        out = []
        while self.pending and len(self.active) < self.max_concurrent:
            if self.policy == SchedulingPolicy.SJF:
                j = min(range(len(self.pending)), key=lambda i: self.pending[i]["remaining"] + self.pending[i]["prompt_len"])
                self.pending.rotate(-j)
                r = self.pending.popleft()
                self.pending.rotate(j)
            else:
                r = self.pending.popleft()
            self.active.append(r)
            out.append(r["id"])
        return out

    def step(self) -> List[int]:
        """One decode iteration: returns the ids that produce a token now (all active; round-robin: one)."""
        self.admit()
        if not self.active:
            return []
        if self.policy == SchedulingPolicy.ROUND_ROBIN:
            self._rr %= len(self.active)
            chosen = [self.active[self._rr]]
            self._rr += 1
        else:
            chosen = list(self.active)
        ids = []
        for r in chosen:
            r["remaining"] -= 1
            ids.append(r["id"])
        self.active = [r for r in self.active if r["remaining"] > 0]
        return ids

    @property
    def idle(self) -> bool:
        return not self.pending and not self.active


class BatchRequestCollector:
    """Collects requests for up to ``window_ms`` or until ``max_batch`` are waiting, then releases them together."""

    def __init__(self, max_batch: int = 4, window_ms: float = 2.0, clock: Callable[[], float] = time.monotonic):
        self.max_batch, self.window, self.clock = max_batch, window_ms / 1e3, clock
        self.items: List[Any] = []
        self.first_at: Optional[float] = None

    def add(self, item) -> Optional[List[Any]]:
        if not self.items:
            self.first_at = self.clock()
        self.items.append(item)
        return self.take() if len(self.items) >= self.max_batch else None

    def poll(self) -> Optional[List[Any]]:
        if self.items and self.clock() - self.first_at >= self.window:
            return self.take()
        return None

    def take(self) -> List[Any]:
        out, self.items, self.first_at = self.items, [], None
        return out
