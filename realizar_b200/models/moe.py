"""Mixture-of-experts: the forward math (router softmax → top-k → renormalise → per-expert
SwiGLU → weighted sum, plus an always-on shared expert) and the serving-side control pieces
(capacity-factor and power-of-two-choices routers, Heijunka load levelling, hot-expert tiers).

The forward groups tokens by expert and runs one GEMM per active expert (tokens sorted by expert
id, contiguous segments), which is the layout an expert-parallel dispatch would exchange.
Reference parity: ``moe_forward`` / ``MoeExpertWeights`` (src/gpu/scheduler/moe_dispatch.rs:10-150,
src/gpu/scheduler/types.rs:117-150); ``CapacityFactorRouter``, ``PowerOfTwoChoicesRouter``,
``HeijunkaController`` (src/moe/mod.rs:25-400); ``ExpertTier`` pinning (src/memory.rs:8-148)."""
from __future__ import annotations

import random
import threading
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class MoeExpertWeights:
    router: torch.Tensor                 # [E, H]
    gate: torch.Tensor                   # [E, I, H]
    up: torch.Tensor                     # [E, I, H]
    down: torch.Tensor                   # [E, H, I]
    shared_gate: Optional[torch.Tensor] = None     # [Is, H]
    shared_up: Optional[torch.Tensor] = None
    shared_down: Optional[torch.Tensor] = None     # [H, Is]
    shared_router: Optional[torch.Tensor] = None   # [1, H] sigmoid gate of the shared expert

    @classmethod
    def random(cls, experts: int, hidden: int, inter: int, shared_inter: int = 0, seed: int = 0, device="cpu", dtype=torch.float32):
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g) * (s[-1] ** -0.5)).to(device=device, dtype=dtype)
        sh = (r(shared_inter, hidden), r(shared_inter, hidden), r(hidden, shared_inter), r(1, hidden)) if shared_inter else (None,) * 4
        return cls(r(experts, hidden), r(experts, inter, hidden), r(experts, inter, hidden), r(experts, hidden, inter), *sh)


def route_topk(x: torch.Tensor, router: torch.Tensor, top_k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` [T, H] → (weights [T, k], expert ids [T, k])."""
    probs = torch.softmax(x.float() @ router.float().t(), dim=-1)
    w, idx = probs.topk(top_k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def moe_forward(x: torch.Tensor, w: MoeExpertWeights, top_k: int, renormalize: bool = True) -> torch.Tensor:
    T, H = x.shape
    wts, idx = route_topk(x, w.router, top_k, renormalize)
    flat_e = idx.reshape(-1)
    order = flat_e.argsort(stable=True)                      # token-slots grouped by expert
    tok = (torch.arange(T * top_k, device=x.device) // top_k)[order]
    counts = torch.bincount(flat_e, minlength=w.router.shape[0]).tolist()
    xs = x[tok]
    ys = torch.empty_like(xs)
    o = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        seg = xs[o:o + c]
        ys[o:o + c] = (F.silu(seg @ w.gate[e].t()) * (seg @ w.up[e].t())) @ w.down[e].t()
        o += c
    out = torch.zeros_like(x)
    out.index_add_(0, tok, ys * wts.reshape(-1)[order].unsqueeze(-1).to(ys.dtype))
    if w.shared_gate is not None:
        sh = (F.silu(x @ w.shared_gate.t()) * (x @ w.shared_up.t())) @ w.shared_down.t()
        if w.shared_router is not None:
            sh = sh * torch.sigmoid(x @ w.shared_router.t())
        out = out + sh
    return out


def moe_forward_reference(x: torch.Tensor, w: MoeExpertWeights, top_k: int, renormalize: bool = True) -> torch.Tensor:
    """Token-by-token restatement used as the oracle in tests."""
    out = torch.zeros_like(x)
    wts, idx = route_topk(x, w.router, top_k, renormalize)
    for t in range(x.shape[0]):
        for j in range(top_k):
            e = int(idx[t, j])
            h = F.silu(w.gate[e] @ x[t]) * (w.up[e] @ x[t])
            out[t] += wts[t, j] * (w.down[e] @ h)
        if w.shared_gate is not None:
            sh = w.shared_down @ (F.silu(w.shared_gate @ x[t]) * (w.shared_up @ x[t]))
            out[t] += sh * (torch.sigmoid(w.shared_router @ x[t]) if w.shared_router is not None else 1.0)
    return out


# -- serving-side routers -------------------------------------------------------------------------
class RouterError(RuntimeError):
    pass


class CapacityFactorRouter:
    """Picks the best-scoring expert replica that still has queue capacity
    (``capacity = ceil(capacity_factor * tokens / experts)``); falls back to the next best."""

    def __init__(self, num_experts: int, capacity: int):
        self.capacity = capacity
        self.load = [0] * num_experts
        self._lock = threading.Lock()

    def route(self, scores: Sequence[float]) -> int:
        if len(scores) != len(self.load):
            raise RouterError(f"expected {len(self.load)} scores, got {len(scores)}")
        with self._lock:
            for e in sorted(range(len(scores)), key=lambda i: -scores[i]):
                if self.load[e] < self.capacity:
                    self.load[e] += 1
                    return e
        raise RouterError("all experts are at capacity")

    def release(self, e: int) -> None:
        with self._lock:
            self.load[e] = max(0, self.load[e] - 1)


class PowerOfTwoChoicesRouter:
    """Sample two candidates, send to the less loaded one: O(1) with near-optimal balance."""

    def __init__(self, num_experts: int, capacity: int, seed: int = 0):
        self.capacity, self.load, self.rng = capacity, [0] * num_experts, random.Random(seed)
        self._lock = threading.Lock()

    def route(self, scores: Optional[Sequence[float]] = None) -> int:
        with self._lock:
            n = len(self.load)
            a, b = self.rng.randrange(n), self.rng.randrange(n)
            if scores is not None and self.load[a] == self.load[b]:
                pick = a if scores[a] >= scores[b] else b
            else:
                pick = a if self.load[a] <= self.load[b] else b
            if self.load[pick] >= self.capacity:
                pick = min(range(n), key=lambda i: self.load[i])
                if self.load[pick] >= self.capacity:
                    raise RouterError("all experts are at capacity")
            self.load[pick] += 1
            return pick

    def release(self, e: int) -> None:
        with self._lock:
            self.load[e] = max(0, self.load[e] - 1)


@dataclass
class HeijunkaController:
    """Load levelling from Little's law: concurrency = arrival rate × latency; requests beyond the
    level that keeps latency at the target are shed."""
    target_latency_ms: float = 100.0
    max_concurrency: int = 64

    def optimal_concurrency(self, arrival_rate_per_s: float, latency_ms: float) -> int:
        return max(1, min(self.max_concurrency, int(round(arrival_rate_per_s * latency_ms / 1e3))))

    def should_shed(self, in_flight: int, observed_latency_ms: float) -> bool:
        return in_flight >= self.max_concurrency or (observed_latency_ms > 2 * self.target_latency_ms and in_flight > 1)

    def level(self, arrival_rate_per_s: float, observed_latency_ms: float) -> dict:
        c = self.optimal_concurrency(arrival_rate_per_s, min(observed_latency_ms, self.target_latency_ms))
        return {"concurrency": c, "shed": observed_latency_ms > 2 * self.target_latency_ms, "utilization": c / self.max_concurrency}


class ExpertTier(Enum):
    HOT = "hot"        # resident on the device
    WARM = "warm"      # pinned host memory
    COLD = "cold"      # pageable / on disk


class ExpertPlacement:
    """Keeps the ``hot_slots`` most used experts on the device, the next ``warm_slots`` in pinned memory."""

    def __init__(self, num_experts: int, hot_slots: int, warm_slots: int = 0):
        self.hits = [0] * num_experts
        self.hot_slots, self.warm_slots = hot_slots, warm_slots

    def record(self, expert_ids: Sequence[int]) -> None:
        for e in expert_ids:
            self.hits[int(e)] += 1

    def tiers(self) -> Dict[int, ExpertTier]:
        order = sorted(range(len(self.hits)), key=lambda e: (-self.hits[e], e))
        return {e: ExpertTier.HOT if r < self.hot_slots else ExpertTier.WARM if r < self.hot_slots + self.warm_slots else ExpertTier.COLD
                for r, e in enumerate(order)}
