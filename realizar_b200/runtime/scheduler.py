"""Request scheduling and the serving loop: continuous batching with mid-batch joins and slot
recycling, KV-aware admission, priorities with aging and deadlines, preemption, chunked prefill
under a per-iteration token budget, and a worker thread that drives an engine and streams tokens
to per-request callbacks.

``Scheduler`` is pure host logic (testable with a fake engine); ``ServingEngine`` binds it to a
``DecodeEngine``.  Capability parity with the reference's scheduling layers: ``Scheduler`` /
``SlotManager`` / ``DynamicPriorityScheduler`` / ``ChunkedPrefillScheduler``
(src/scheduler/mod_max_scheduler.rs:4-460, src/scheduler/mod_dynamic_scheduler.rs:34-400,
src/scheduler/chunked_prefill.rs:26-370), the CUDA batch scheduler thread with joins and recycling
(src/api/cuda_batch_scheduler.rs:94-460) and the iteration scheduler (src/api/iteration_scheduler.rs:1-80).
"""
from __future__ import annotations

import itertools
import logging
import queue
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Deque, Dict, List, Optional, Sequence

log = logging.getLogger("realizar_b200.scheduler")


class RequestState(Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"


class FinishReason(Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    ERROR = "error"


@dataclass
class Request:
    prompt: List[int]
    max_tokens: int = 64
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    stop_token_ids: Sequence[int] = ()
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Optional[Dict[int, float]] = None
    token_masker: Optional[object] = None  # grammar / tool-call constraint: ``mask() -> bool[vocab]`` and ``accept_token(id)``
    stop_check: Optional[Callable[["Request"], bool]] = None   # called after every token; True ends the request (stop strings)
    priority: int = 0                      # larger = more urgent
    deadline: Optional[float] = None       # absolute time.monotonic() deadline
    on_token: Optional[Callable[[int], None]] = None
    on_finish: Optional[Callable[["Request"], None]] = None
    id: int = field(default_factory=itertools.count().__next__)
    arrival: float = field(default_factory=time.monotonic)
    state: RequestState = RequestState.WAITING
    output: List[int] = field(default_factory=list)
    prefilled: int = 0                     # prompt tokens already in the KV cache
    slot: int = -1
    finish_reason: Optional[FinishReason] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    error: Optional[str] = None
    cancelled: bool = False

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival


@dataclass
class SchedulerConfig:
    max_batch: int = 4
    max_seq_len: int = 2048
    max_waiting: int = 1024                # queue bound: beyond it add_request refuses (HTTP 503 upstream)
    token_budget: int = 512                # prompt tokens + decode tokens per iteration
    prefill_chunk: int = 256
    max_prefills_per_iter: int = 1
    aging_seconds: float = 5.0             # a waiting request gains one priority level per this many seconds
    allow_preemption: bool = True
    policy: str = "priority"               # "priority" | "fcfs" | "sjf"


@dataclass
class ScheduleDecision:
    prefill: List[tuple] = field(default_factory=list)      # (request, start, end) prompt chunk
    decode: List[Request] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    admitted: List[Request] = field(default_factory=list)


class QueueFull(RuntimeError):
    pass


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, page_size: int = 16, total_pages: Optional[int] = None):
        self.cfg = cfg
        self.page_size = page_size
        self.total_pages = total_pages if total_pages is not None else cfg.max_batch * (-(-cfg.max_seq_len // page_size))
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.preempted: Deque[Request] = deque()
        self.free_slots: List[int] = list(range(cfg.max_batch - 1, -1, -1))
        self.pages_in_use = 0
        self.stats = {"admitted": 0, "finished": 0, "preemptions": 0, "rejected": 0, "iterations": 0, "tokens": 0}

    # -- queueing ----------------------------------------------------------------------------
    def add_request(self, r: Request) -> Request:
        if len(r.prompt) == 0:
            raise ValueError("empty prompt")
        if len(r.prompt) + 1 > self.cfg.max_seq_len:
            raise ValueError(f"prompt of {len(r.prompt)} tokens exceeds the context length {self.cfg.max_seq_len}")
        if len(self.waiting) >= self.cfg.max_waiting:
            self.stats["rejected"] += 1
            raise QueueFull("request queue is full")
        r.max_tokens = max(1, min(r.max_tokens, self.cfg.max_seq_len - len(r.prompt)))
        self.waiting.append(r)
        return r

    def _pages(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def _effective_priority(self, r: Request, now: float) -> float:
        p = r.priority + (now - r.arrival) / max(1e-6, self.cfg.aging_seconds)
        if r.deadline is not None:
            p += max(0.0, 10.0 - max(0.0, r.deadline - now))       # urgency grows as the deadline nears
        return p

    def _pick_waiting(self, now: float) -> Optional[Request]:
        pool = list(self.preempted) + list(self.waiting)
        if not pool:
            return None
        if self.cfg.policy == "fcfs":
            return min(pool, key=lambda r: r.arrival)
        if self.cfg.policy == "sjf":
            return min(pool, key=lambda r: (len(r.prompt) + r.max_tokens, r.arrival))
        return max(pool, key=lambda r: (self._effective_priority(r, now), -r.arrival))

    def _remove_from_queues(self, r: Request) -> None:
        for q in (self.waiting, self.preempted):
            try:
                q.remove(r)
                return
            except ValueError:
                pass

    # -- one iteration -------------------------------------------------------------------------
    def schedule(self, now: Optional[float] = None) -> ScheduleDecision:
        now = time.monotonic() if now is None else now
        d = ScheduleDecision()
        self.stats["iterations"] += 1
        # 1. admit while there is a slot and KV room for prompt + max_tokens
        while self.free_slots:
            r = self._pick_waiting(now)
            if r is None:
                break
            need = self._pages(len(r.prompt) + len(r.output) + r.max_tokens)
            if self.pages_in_use + need > self.total_pages:
                victim = self._preemption_victim(r, now) if self.cfg.allow_preemption else None
                if victim is None:
                    break
                self._preempt(victim)
                d.preempted.append(victim)
                continue
            self._remove_from_queues(r)
            r.slot = self.free_slots.pop()
            r.state = RequestState.PREFILL
            r.prefilled = 0
            self.pages_in_use += need
            r._pages = need
            self.running.append(r)
            d.admitted.append(r)
            self.stats["admitted"] += 1
        # 2. decode-maximal batching: every running sequence past its prompt decodes one token
        budget = self.cfg.token_budget
        for r in self.running:
            if r.state == RequestState.RUNNING:
                d.decode.append(r)
                budget -= 1
        # 3. fill the remaining budget with prompt chunks
        n_pref = 0
        for r in self.running:
            if r.state != RequestState.PREFILL or n_pref >= self.cfg.max_prefills_per_iter or budget <= 0:
                continue
            full = r.prompt + r.output                   # a preempted request re-prefills what it had generated
            start = r.prefilled
            end = min(len(full), start + min(self.cfg.prefill_chunk, budget))
            if end > start:
                d.prefill.append((r, start, end))
                budget -= end - start
                n_pref += 1
        return d

    def _preemption_victim(self, incoming: Request, now: float) -> Optional[Request]:
        cand = [r for r in self.running if r.priority < incoming.priority]
        return min(cand, key=lambda r: (r.priority, -r.arrival)) if cand else None

    def _preempt(self, r: Request) -> None:
        self.running.remove(r)
        self.free_slots.append(r.slot)
        self.pages_in_use -= getattr(r, "_pages", 0)
        r.state, r.slot, r.prefilled = RequestState.PREEMPTED, -1, 0
        self.preempted.append(r)
        self.stats["preemptions"] += 1

    # -- results -------------------------------------------------------------------------------
    def on_prefill_done(self, r: Request, end: int, first_token: Optional[int], now: Optional[float] = None) -> None:
        r.prefilled = end
        if end >= len(r.prompt) + len(r.output) and first_token is not None:
            r.state = RequestState.RUNNING
            self.on_token(r, first_token, now)

    def on_token(self, r: Request, token: int, now: Optional[float] = None) -> None:
        now = time.monotonic() if now is None else now
        r.output.append(int(token))
        r.token_times.append(now)
        self.stats["tokens"] += 1
        if r.first_token_time is None:
            r.first_token_time = now
        if r.on_token is not None:
            try:
                r.on_token(int(token))
            except Exception as e:                         # a broken consumer must not take the loop down
                log.warning("on_token callback failed: %s", e)
                r.cancelled = True
        if r.cancelled:
            self.finish(r, FinishReason.ABORT, now)
        elif int(token) in r.stop_token_ids:
            self.finish(r, FinishReason.STOP, now)
        elif len(r.output) >= r.max_tokens or r.total_len >= self.cfg.max_seq_len:
            self.finish(r, FinishReason.LENGTH, now)

    def finish(self, r: Request, reason: FinishReason, now: Optional[float] = None, error: Optional[str] = None) -> None:
        if r.state == RequestState.FINISHED:
            return
        if r in self.running:
            self.running.remove(r)
            self.free_slots.append(r.slot)
            self.pages_in_use -= getattr(r, "_pages", 0)
        else:
            self._remove_from_queues(r)
        r.state, r.finish_reason, r.error = RequestState.FINISHED, reason, error
        r.finish_time = time.monotonic() if now is None else now
        self.stats["finished"] += 1
        if getattr(self, "on_finished", None) is not None:   # the owner's per-request accounting
            self.on_finished(r)
        if r.on_finish is not None:
            try:
                r.on_finish(r)
            except Exception as e:
                log.warning("on_finish callback failed: %s", e)

    def abort(self, request_id: int) -> bool:
        for r in list(self.running) + list(self.waiting) + list(self.preempted):
            if r.id == request_id:
                r.cancelled = True
                if r.state in (RequestState.WAITING, RequestState.PREEMPTED):
                    self.finish(r, FinishReason.ABORT)
                return True
        return False

    @property
    def has_work(self) -> bool:
        return bool(self.running or self.waiting or self.preempted)

    def snapshot(self) -> dict:
        return {"waiting": len(self.waiting), "running": len(self.running), "preempted": len(self.preempted),
                "free_slots": len(self.free_slots), "kv_page_utilization": self.pages_in_use / max(1, self.total_pages), **self.stats}


class ServingEngine:
    """Owns the engine on one worker thread: admits requests, runs prompt chunks and batched decode
    steps, streams tokens through callbacks.  ``health`` turns to "unhealthy" when a step raises
    (a circuit-breaker style latch that the API layer reports as 503)."""

    def __init__(self, engine, cfg: Optional[SchedulerConfig] = None, idle_sleep: float = 0.001, draft_layers: Optional[Sequence[int]] = None,
                 spec_k: int = 4):
        self.engine = engine
        self.draft_layers = tuple(draft_layers) if draft_layers else None
        self.spec_k = spec_k
        self.spec_stats = {"rounds": 0, "drafted": 0, "accepted": 0}
        ecfg = engine.cfg
        self.cfg = cfg or SchedulerConfig(max_batch=ecfg.max_batch, max_seq_len=ecfg.max_seq_len)
        self.sched = Scheduler(self.cfg, total_pages=getattr(engine, "num_pages", None))
        self._inbox: "queue.Queue[Request]" = queue.Queue()
        self._calls: "queue.Queue" = queue.Queue()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.idle_sleep = idle_sleep
        self.health = "ok"
        self.last_error: Optional[str] = None
        self.step_times: Deque[float] = deque(maxlen=512)
        self._lock = threading.Lock()
        from .batch_types import InferenceEventNotifier, InferenceMetrics
        self.inference = InferenceMetrics()                  # per-request latency / token counters (reported by metrics())
        self.notifier = InferenceEventNotifier()             # callbacks (request id, latency ms, tokens) at the end of every request
        self.notifier.register(lambda _rid, ms, n: self.inference.record(ms, n))
        self.sched.on_finished = self._request_finished

    def _request_finished(self, r: "Request") -> None:
        self.notifier.notify(r.id, 1e3 * (time.monotonic() - r.arrival), len(r.output))

    # -- public ---------------------------------------------------------------------------------
    def start(self) -> "ServingEngine":
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop, name="realizar-engine", daemon=True)
            self._thread.start()
        return self

    def stop(self, timeout: float = 5.0) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout)
            self._thread = None

    def submit(self, r: Request) -> Request:
        if self.health != "ok":
            raise RuntimeError(f"engine is {self.health}: {self.last_error}")
        with self._lock:
            if self._inbox.qsize() + len(self.sched.waiting) >= self.cfg.max_waiting:
                self.sched.stats["rejected"] += 1
                raise QueueFull("request queue is full")
        self._inbox.put(r)
        return r

    def call_on_engine(self, fn: Callable[[object], object], timeout: Optional[float] = 120.0):
        """Run ``fn(engine)`` on the engine thread between two scheduling iterations and return its result (scoring passes,
        KV snapshots: anything that needs the engine while requests are being served)."""
        if self.health != "ok":
            raise RuntimeError(f"engine is {self.health}: {self.last_error}")
        from .batch_types import AsyncGpuResult
        res = AsyncGpuResult()

        def job(engine):
            try:
                res.set_result(fn(engine))
            except Exception as e:                           # delivered to the caller, the serving loop goes on
                res.set_error(e)
        if self._thread is None:                             # no worker thread (tests that drive step() themselves)
            job(self.engine)
        else:
            self._calls.put(job)
        return res.wait(timeout)                             # TimeoutError when the loop did not get to it in time

    def generate(self, prompt: Sequence[int], timeout: Optional[float] = None, **kw) -> Request:
        """Blocking convenience: submit and wait for completion."""
        done = threading.Event()
        r = Request(list(prompt), on_finish=lambda _r: done.set(), **kw)
        self.submit(r)
        if not done.wait(timeout):
            r.cancelled = True
            raise TimeoutError("generation timed out")
        return r

    # -- loop -------------------------------------------------------------------------------------
    def _drain_inbox(self) -> None:
        while True:
            try:
                r = self._inbox.get_nowait()
            except queue.Empty:
                return
            try:
                self.sched.add_request(r)
            except Exception as e:
                r.error = str(e)
                r.state, r.finish_reason = RequestState.FINISHED, FinishReason.ERROR
                if r.on_finish:
                    r.on_finish(r)

    def step(self) -> bool:
        """One scheduling iteration.  Returns False when there was nothing to do."""
        self._drain_inbox()
        ran_call = False
        while True:                                          # engine calls queued by other threads (scoring, snapshots)
            try:
                job = self._calls.get_nowait()
            except queue.Empty:
                break
            job(self.engine)
            ran_call = True
        if not self.sched.has_work:
            return ran_call
        t0 = time.monotonic()
        d = self.sched.schedule()
        eng = self.engine
        for r in d.preempted:
            eng.close_slot(getattr(r, "_engine_slot", -1)) if getattr(r, "_engine_slot", -1) >= 0 else None
            r._engine_slot = -1
        for r in d.admitted:
            eng.open_slot(r.slot, min(self.cfg.max_seq_len, len(r.prompt) + len(r.output) + r.max_tokens))
            from .engine import SamplingParams
            eng.set_sampling(r.slot, SamplingParams(r.temperature, r.top_k, r.top_p, r.min_p, r.max_tokens,
                                                    repetition_penalty=r.repetition_penalty, presence_penalty=r.presence_penalty,
                                                    frequency_penalty=r.frequency_penalty, logit_bias=r.logit_bias))
            if r.token_masker is not None:
                eng.set_token_mask(r.slot, r.token_masker.mask())
            r._engine_slot = r.slot
        # decode first (latency of running streams), then prompt chunks
        live = [r for r in d.decode if not r.cancelled]
        for r in d.decode:
            if r.cancelled:
                self._finish(r, FinishReason.ABORT)
        if live and self._speculative_round(live):
            pass
        elif live:
            out = eng.feed({r.slot: r.output[-1] for r in live})
            now = time.monotonic()
            for r in live:
                slot = r.slot
                self._emit(r, int(out[slot]), now)
                if r.state == RequestState.FINISHED:
                    eng.close_slot(slot)
        for r, start, end in d.prefill:
            if r.cancelled:
                self._finish(r, FinishReason.ABORT)
                continue
            slot = r.slot
            full = r.prompt + r.output
            tok = eng.prefill(slot, full[start:end])
            last = end >= len(full)
            self.sched.on_prefill_done(r, end, tok if last else None)
            if last and r.state != RequestState.FINISHED:
                self._after_token(r, int(tok))
            if r.state == RequestState.FINISHED:
                eng.close_slot(slot)
        self.step_times.append(time.monotonic() - t0)
        return True

    def _emit(self, r: Request, tok: int, now: float) -> None:
        """A decode step produced ``tok`` for ``r``: scheduler bookkeeping, then the request's own constraints."""
        self.sched.on_token(r, tok, now)
        if r.state != RequestState.FINISHED:
            self._after_token(r, tok)

    def _after_token(self, r: Request, tok: int) -> None:
        """Grammar state and stop strings after a token; the mask for the NEXT token goes to the device."""
        if r.token_masker is not None:
            r.token_masker.accept_token(tok)
            self.engine.set_token_mask(r.slot, r.token_masker.mask())
        if r.stop_check is not None and r.stop_check(r):
            self.sched.finish(r, FinishReason.STOP)

    def _speculative_round(self, live) -> bool:
        """Self-speculative decoding for a lone greedy stream (server option ``draft_layers``): the layer-skipping draft
        proposes ``spec_k`` tokens, one tensor-core pass of the full model checks them, and the agreeing prefix plus the
        model's own next token are emitted - between 1 and ``spec_k + 1`` tokens for one read of the weights.
        Returns False when the step has to run normally."""
        if not self.draft_layers or len(live) != 1:
            return False
        r, eng = live[0], self.engine
        if (r.slot != 0 or r.temperature > 0 or r.token_masker is not None or r.logit_bias or r.repetition_penalty != 1.0
                or r.presence_penalty or r.frequency_penalty or not getattr(eng, "gemm_ok", False)):
            return False
        from .batch_types import SpeculativeBuffer
        from .speculative import verify_greedy
        k = min(self.spec_k, r.max_tokens - len(r.output) - 1, self.cfg.max_seq_len - r.total_len - 2)
        if k < 1:
            return False
        pos0 = eng.slots[0].position
        last, feed, buf = r.output[-1], r.output[-1], SpeculativeBuffer(capacity=k)
        for _ in range(k):
            feed = eng.draft_step(0, int(feed), self.draft_layers)
            buf.add_candidate(int(feed), 1.0)
        drafts = [t for t, _ in buf.items]
        eng.rollback(0, pos0)
        nxt = eng.forward_tokens(0, [last] + drafts)
        v = verify_greedy(drafts, nxt)
        assert buf.verify(nxt)[0] == v.accepted
        eng.rollback(0, pos0 + 1 + v.accepted)
        self.spec_stats["rounds"] += 1
        self.spec_stats["drafted"] += k
        self.spec_stats["accepted"] += v.accepted
        now = time.monotonic()
        for t in v.tokens:
            self._emit(r, int(t), now)
            if r.state == RequestState.FINISHED:
                eng.close_slot(0)
                break
        return True                                          # the last emitted token has not been fed yet, exactly as after feed()

    def _finish(self, r: Request, reason: FinishReason) -> None:
        slot = r.slot
        self.sched.finish(r, reason)
        if slot >= 0:
            self.engine.close_slot(slot)

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                if not self.step():
                    time.sleep(self.idle_sleep)
            except Exception as e:                          # latch unhealthy, fail everything in flight
                log.exception("engine step failed")
                self.health, self.last_error = "unhealthy", repr(e)
                for r in list(self.sched.running) + list(self.sched.waiting) + list(self.sched.preempted):
                    self.sched.finish(r, FinishReason.ERROR, error=repr(e))
                return

    def recover(self) -> bool:
        """After the loop latched unhealthy: probe the engine and, when it still answers, bring the server back.  Everything
        that was in flight has already been failed; ``engine.reset()`` returns the engine to its post-load state (no open
        sequences, error words cleared) and must raise when the device context itself is lost - then the process has to be
        restarted and the latch stays.  Returns True when serving again.  (Role of the reference's poisoned-context detection
        and pool reset, src/cuda/executor/mod.rs:60-118.)"""
        if self.health == "ok":
            return True
        if self._thread is not None and self._thread.is_alive():
            return False                                     # the loop has not finished failing its requests yet
        try:
            reset = getattr(self.engine, "reset", None)
            if reset is None:
                raise RuntimeError("the engine cannot be reset in place")
            reset()
        except Exception as e:                               # context lost (or no reset path): stay latched
            self.last_error = f"recovery failed: {e!r}"
            return False
        self.sched = Scheduler(self.cfg, total_pages=getattr(self.engine, "num_pages", None))
        self.sched.on_finished = self._request_finished
        while not self._inbox.empty():                       # requests that slipped in between the failure and the latch
            try:
                r = self._inbox.get_nowait()
                r.error, r.state, r.finish_reason = "engine was reset", RequestState.FINISHED, FinishReason.ERROR
                if r.on_finish:
                    r.on_finish(r)
            except queue.Empty:
                break
        self.health, self.last_error = "ok", None
        self._thread = None
        self._stop.clear()
        self.start()
        return True

    def metrics(self) -> dict:
        st = list(self.step_times)
        snap = self.sched.snapshot()
        snap.update({"health": self.health, "avg_step_ms": 1e3 * sum(st) / len(st) if st else 0.0, "queue_depth": self._inbox.qsize() + snap["waiting"],
                     "requests_done": self.inference.total_inferences, "request_latency_ms_p50": self.inference.percentile(50),
                     "request_latency_ms_p99": self.inference.percentile(99)})
        return snap


class FakeEngine:
    """Engine stand-in for host-side tests: the token after ``t`` is ``(t + 1) % vocab``; a request ends
    when it emits ``eos``.  Records the calls it receives."""

    @dataclass
    class Cfg:
        max_batch: int = 4
        max_seq_len: int = 256

    def __init__(self, max_batch: int = 4, max_seq_len: int = 256, vocab: int = 100, fail_after: Optional[int] = None):
        self.cfg = FakeEngine.Cfg(max_batch, max_seq_len)
        self.vocab, self.calls, self.open, self.fail_after, self.steps = vocab, [], {}, fail_after, 0
        self.num_pages = max_batch * (-(-max_seq_len // 16))

    def open_slot(self, slot, reserve):
        assert slot not in self.open, f"slot {slot} reused while busy"
        self.open[slot] = 0
        self.calls.append(("open", slot, reserve))

    def close_slot(self, slot):
        self.open.pop(slot, None)
        getattr(self, "masks", {}).pop(slot, None)
        self.calls.append(("close", slot))

    def set_sampling(self, slot, sp):
        self.calls.append(("sampling", slot, sp.temperature))
        self.sampling = getattr(self, "sampling", {})
        self.sampling[slot] = sp
        self.sampling_log = getattr(self, "sampling_log", [])
        self.sampling_log.append(sp)

    def set_token_mask(self, slot, allowed):
        self.masks = getattr(self, "masks", {})
        self.masks[slot] = None if allowed is None else [int(i) for i, a in enumerate(allowed) if a]
        self.calls.append(("mask", slot, None if allowed is None else int(sum(bool(a) for a in allowed))))

    def free_slots(self):
        return [i for i in range(self.cfg.max_batch) if i not in self.open]

    def reset(self) -> None:
        """Back to the post-load state (``fail_after`` counts from here again; ``context_lost`` makes the probe fail)."""
        if getattr(self, "context_lost", False):
            raise RuntimeError("device context lost")
        self.open.clear()
        self.steps = 0

    def score_tokens(self, tokens, want_embedding=False, top_k=0):
        """Scores of the toy model: the successor (t + 1) % vocab has probability 1/2."""
        import math
        self.calls.append(("score", len(tokens)))
        lps = [math.log(0.5) if b == (a + 1) % self.vocab else math.log(0.5 / (self.vocab - 1)) for a, b in zip(tokens, tokens[1:])]
        out = {"logprobs": lps, "num_tokens": len(tokens)}
        if lps:
            out["nll"] = -sum(lps) / len(lps)
            out["perplexity"] = math.exp(out["nll"])
        if want_embedding:
            out["embedding"] = [float(sum(tokens)) / len(tokens), float(len(tokens))]
        return out

    def prefill(self, slot, tokens):
        self.open[slot] += len(tokens)
        self.calls.append(("prefill", slot, len(tokens)))
        return self._pick(slot, (int(tokens[-1]) + 1) % self.vocab)

    def feed(self, slot_tokens):
        self.steps += 1
        if self.fail_after is not None and self.steps > self.fail_after:
            raise RuntimeError("injected engine failure")
        self.calls.append(("feed", tuple(sorted(slot_tokens))))
        out = [0] * self.cfg.max_batch
        for s, t in slot_tokens.items():
            self.open[s] += 1
            out[s] = self._pick(s, (int(t) + 1) % self.vocab)
        return out

    def _pick(self, slot, default):
        """A token mask restricts the fake's choice: the default if it is allowed, else the smallest allowed id."""
        allowed = getattr(self, "masks", {}).get(slot)
        if allowed is None or default in allowed or not allowed:
            return default
        return allowed[0]
