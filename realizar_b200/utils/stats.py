"""Benchmark statistics: descriptive summaries, Welch's t-test, Mann-Whitney U, bootstrap
confidence intervals and effect sizes, used to decide whether two runs differ.
Reference parity: src/stats.rs:24-417 (``analyze_with_auto_select``, ``TestMethod``, ``AnalysisResult``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import numpy as np


@dataclass
class Summary:
    n: int
    mean: float
    std: float
    min: float
    max: float
    p50: float
    p95: float
    p99: float
    cv: float


def summarize(xs: Sequence[float]) -> Summary:
    a = np.asarray(xs, np.float64)
    if a.size == 0:
        return Summary(0, 0, 0, 0, 0, 0, 0, 0, 0)
    m, s = float(a.mean()), float(a.std(ddof=1)) if a.size > 1 else 0.0
    return Summary(int(a.size), m, s, float(a.min()), float(a.max()), *(float(np.percentile(a, q)) for q in (50, 95, 99)), s / m if m else 0.0)


def _t_sf(t: float, df: float) -> float:
    """Two-sided p-value of Student's t via the regularised incomplete beta function."""
    from scipy.special import betainc
    x = df / (df + t * t)
    return float(betainc(df / 2.0, 0.5, x))


@dataclass
class TestResult:
    method: str
    statistic: float
    p_value: float
    effect_size: float
    significant: bool


def welch_t_test(a: Sequence[float], b: Sequence[float], alpha: float = 0.05) -> TestResult:
    x, y = np.asarray(a, np.float64), np.asarray(b, np.float64)
    vx, vy = x.var(ddof=1) / x.size, y.var(ddof=1) / y.size
    se = math.sqrt(vx + vy)
    if se == 0:
        same = float(x.mean()) == float(y.mean())
        return TestResult("welch", 0.0 if same else math.inf, 1.0 if same else 0.0, 0.0, not same)
    t = float((x.mean() - y.mean()) / se)
    df = (vx + vy) ** 2 / (vx ** 2 / (x.size - 1) + vy ** 2 / (y.size - 1))
    p = _t_sf(abs(t), df)
    pooled = math.sqrt((x.var(ddof=1) + y.var(ddof=1)) / 2)
    return TestResult("welch", t, p, float((x.mean() - y.mean()) / pooled) if pooled else 0.0, p < alpha)


def mann_whitney_u(a: Sequence[float], b: Sequence[float], alpha: float = 0.05) -> TestResult:
    x, y = np.asarray(a, np.float64), np.asarray(b, np.float64)
    allv = np.concatenate([x, y])
    order = allv.argsort(kind="mergesort")
    ranks = np.empty_like(allv)
    sv = allv[order]
    i = 0
    tie_term = 0.0
    while i < sv.size:
        j = i
        while j + 1 < sv.size and sv[j + 1] == sv[i]:
            j += 1
        ranks[order[i:j + 1]] = (i + j) / 2 + 1
        t = j - i + 1
        tie_term += t ** 3 - t
        i = j + 1
    n1, n2 = x.size, y.size
    u1 = ranks[:n1].sum() - n1 * (n1 + 1) / 2
    u = min(u1, n1 * n2 - u1)
    n = n1 + n2
    sigma = math.sqrt(n1 * n2 / 12 * ((n + 1) - tie_term / (n * (n - 1)))) if n > 1 else 0.0
    if sigma == 0:
        return TestResult("mann-whitney", float(u), 1.0, 0.0, False)
    z = (u - n1 * n2 / 2 + 0.5) / sigma
    p = math.erfc(abs(z) / math.sqrt(2))
    return TestResult("mann-whitney", float(u), float(p), float(1 - 2 * u / (n1 * n2)), p < alpha)


def is_roughly_normal(xs: Sequence[float]) -> bool:
    a = np.asarray(xs, np.float64)
    if a.size < 8 or a.std() == 0:
        return a.size >= 8
    z = (a - a.mean()) / a.std()
    return abs(float((z ** 3).mean())) < 1.0 and abs(float((z ** 4).mean()) - 3.0) < 2.0


def analyze_with_auto_select(a: Sequence[float], b: Sequence[float], alpha: float = 0.05) -> TestResult:
    """Welch when both samples look normal, Mann-Whitney otherwise."""
    return welch_t_test(a, b, alpha) if is_roughly_normal(a) and is_roughly_normal(b) else mann_whitney_u(a, b, alpha)


def bootstrap_ci(xs: Sequence[float], stat=np.mean, n_boot: int = 2000, level: float = 0.95, seed: int = 0):
    a = np.asarray(xs, np.float64)
    rng = np.random.default_rng(seed)
    vals = np.array([stat(a[rng.integers(0, a.size, a.size)]) for _ in range(n_boot)])
    lo, hi = np.percentile(vals, [(1 - level) / 2 * 100, (1 + level) / 2 * 100])
    return float(lo), float(hi)
