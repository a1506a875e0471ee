"""Compute bricks: each stage of the token pipeline as an object with a time budget per token,
assertions on its output, and a verification report; a layer is a list of bricks, and the layer
report names the bottleneck.  Budgets derive from the roofline: a stage that moves ``bytes`` through
HBM cannot be faster than ``bytes / bandwidth``.  Reference parity: ``ComputeBrick`` /
``TokenBudget`` / ``BrickAssertion`` / ``BrickVerification`` / ``TransformerLayerBrick`` /
``BottleneckReport`` (src/brick/*.rs)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np


@dataclass
class TokenBudget:
    us_per_token: float

    @classmethod
    def from_throughput(cls, tok_per_s: float) -> "TokenBudget":
        return cls(1e6 / tok_per_s)

    @classmethod
    def from_bytes(cls, nbytes: float, bandwidth_gbs: float, efficiency: float = 1.0) -> "TokenBudget":
        return cls(nbytes / (bandwidth_gbs * 1e3 * efficiency))

    @property
    def tok_per_s(self) -> float:
        return 1e6 / self.us_per_token

    def is_met(self, actual_us: float) -> bool:
        return actual_us <= self.us_per_token

    def gap_factor(self, actual_us: float) -> float:
        return actual_us / self.us_per_token


@dataclass
class BrickAssertion:
    name: str
    kind: str                     # "no_nan" | "bounds" | "equiv" | "budget" | "custom"
    lo: float = -np.inf
    hi: float = np.inf
    tolerance: float = 1e-3
    fn: Optional[Callable[[np.ndarray], bool]] = None

    def check(self, out: np.ndarray, reference: Optional[np.ndarray] = None) -> bool:
        a = np.asarray(out, np.float64)
        if self.kind == "no_nan":
            return bool(np.isfinite(a).all())
        if self.kind == "bounds":
            return bool((a >= self.lo).all() and (a <= self.hi).all())
        if self.kind == "equiv":
            return reference is not None and bool(np.abs(a - np.asarray(reference, np.float64)).max() <= self.tolerance)
        if self.kind == "custom":
            return bool(self.fn(a))
        return True


@dataclass
class BrickVerification:
    brick: str
    passed: bool
    failures: List[str] = field(default_factory=list)
    actual_us: Optional[float] = None
    budget_us: Optional[float] = None


class ComputeBrick:
    def __init__(self, name: str, budget: TokenBudget, run: Optional[Callable[..., np.ndarray]] = None, assertions: Optional[List[BrickAssertion]] = None,
                 bytes_moved: int = 0, flops: int = 0):
        self.name, self.budget, self.run_fn = name, budget, run
        self.assertions = assertions if assertions is not None else [BrickAssertion("finite", "no_nan")]
        self.bytes_moved, self.flops = bytes_moved, flops
        self.last_us: Optional[float] = None

    def record(self, us: float) -> None:
        self.last_us = us

    def verify(self, out=None, reference=None) -> BrickVerification:
        fails = [a.name for a in self.assertions if out is not None and not a.check(out, reference)]
        if self.last_us is not None and not self.budget.is_met(self.last_us):
            fails.append(f"budget ({self.last_us:.2f}us > {self.budget.us_per_token:.2f}us)")
        return BrickVerification(self.name, not fails, fails, self.last_us, self.budget.us_per_token)

    def achieved_gbs(self) -> Optional[float]:
        return self.bytes_moved / (self.last_us * 1e3) if self.last_us else None


@dataclass
class BottleneckReport:
    brick: str
    actual_us: float
    budget_us: float
    share: float

    @property
    def gap(self) -> float:
        return self.actual_us / self.budget_us


class TransformerLayerBrick:
    """The decode pipeline of one layer: RmsNorm, Qkv, Rope, Attention, OProj, Ffn (+ residuals)."""

    STAGES = ("RmsNorm", "QkvProjection", "RopeEmbedding", "AttentionScore", "OutputProjection", "GateUpProjection", "DownProjection", "Residual")

    def __init__(self, bricks: List[ComputeBrick]):
        self.bricks = bricks

    @classmethod
    def from_model_shape(cls, hidden: int, q_dim: int, kv_dim: int, inter: int, bits_per_weight: float, context: int, bandwidth_gbs: float,
                         efficiency: float = 0.5, gated: bool = True) -> "TransformerLayerBrick":
        wb = lambda n, k: int(n * k * bits_per_weight / 8)
        mk = lambda name, b: ComputeBrick(name, TokenBudget.from_bytes(max(b, 1), bandwidth_gbs, efficiency), bytes_moved=b)
        return cls([mk("RmsNorm", 8 * hidden), mk("QkvProjection", wb(q_dim + 2 * kv_dim, hidden)), mk("RopeEmbedding", 8 * (q_dim + kv_dim)),
                    mk("AttentionScore", 2 * 2 * kv_dim * context), mk("OutputProjection", wb(hidden, q_dim)),
                    mk("GateUpProjection", wb((2 if gated else 1) * inter, hidden)), mk("DownProjection", wb(hidden, inter)), mk("Residual", 12 * hidden)])

    def total_budget_us(self) -> float:
        return sum(b.budget.us_per_token for b in self.bricks)

    def total_actual_us(self) -> float:
        return sum(b.last_us or 0.0 for b in self.bricks)

    def record(self, timings_us: Dict[str, float]) -> None:
        for b in self.bricks:
            if b.name in timings_us:
                b.record(timings_us[b.name])

    def bottleneck(self) -> Optional[BottleneckReport]:
        timed = [b for b in self.bricks if b.last_us]
        if not timed:
            return None
        tot = sum(b.last_us for b in timed)
        w = max(timed, key=lambda b: b.last_us - b.budget.us_per_token)
        return BottleneckReport(w.name, w.last_us, w.budget.us_per_token, w.last_us / tot)

    def verify(self) -> List[BrickVerification]:
        return [b.verify() for b in self.bricks]
