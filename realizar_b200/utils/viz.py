"""Terminal visualisation of benchmark data: sparklines, ASCII histograms, bar tables.
Reference parity: src/viz.rs:24-449 (``sparkline``, ``histogram``, ``BenchmarkData::print_full_report``)."""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np

from .stats import summarize

_TICKS = "▁▂▃▄▅▆▇█"


def sparkline(xs: Sequence[float], width: int = 0) -> str:
    a = np.asarray(xs, np.float64)
    if a.size == 0:
        return ""
    if width and a.size > width:
        a = np.array([c.mean() for c in np.array_split(a, width)])
    lo, hi = float(a.min()), float(a.max())
    if hi == lo:
        return _TICKS[0] * a.size
    return "".join(_TICKS[min(7, int((v - lo) / (hi - lo) * 8))] for v in a)


def histogram(xs: Sequence[float], bins: int = 10, width: int = 40, unit: str = "") -> str:
    a = np.asarray(xs, np.float64)
    if a.size == 0:
        return "(no data)"
    counts, edges = np.histogram(a, bins=bins)
    top = max(1, counts.max())
    return "\n".join(f"{edges[i]:>10.3f}-{edges[i + 1]:<10.3f}{unit} |{'█' * int(round(c / top * width))} {c}" for i, c in enumerate(counts))


def bar_table(rows: Dict[str, float], width: int = 40, unit: str = "") -> str:
    if not rows:
        return "(no data)"
    top = max(rows.values()) or 1.0
    w = max(len(k) for k in rows)
    return "\n".join(f"{k:<{w}} |{'█' * int(round(v / top * width))} {v:.2f}{unit}" for k, v in rows.items())


def full_report(name: str, xs: Sequence[float], unit: str = "ms") -> str:
    s = summarize(xs)
    return (f"== {name} ==\n n={s.n} mean={s.mean:.3f}{unit} std={s.std:.3f} cv={100 * s.cv:.1f}% min={s.min:.3f} p50={s.p50:.3f} "
            f"p95={s.p95:.3f} p99={s.p99:.3f} max={s.max:.3f}\n trend {sparkline(xs, 60)}\n{histogram(xs, unit=unit)}")
