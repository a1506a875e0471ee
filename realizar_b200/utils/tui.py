"""Terminal monitor: polls the server's ``/v1/metrics`` and renders throughput (sparkline),
latency percentiles, queue depth, batch occupancy and GPU memory.
Reference parity: ``realizar-monitor`` (src/bin/realizar_monitor/main.rs:1-60), ``InferenceTui`` (src/tui.rs:43-332)."""
from __future__ import annotations

import json
import time
import urllib.request
from collections import deque
from typing import Deque, Optional

from .viz import sparkline


class MonitorState:
    def __init__(self, history: int = 60):
        self.tps: Deque[float] = deque(maxlen=history)
        self.last: dict = {}
        self.errors = 0

    def update(self, m: dict) -> None:
        self.last = m
        self.tps.append(float(m.get("tokens_per_sec", m.get("throughput_tok_s", 0.0)) or 0.0))

    def render(self, width: int = 72) -> str:
        m = self.last
        g = lambda *ks, d=0: next((m[k] for k in ks if k in m), d)
        bar = "─" * width
        lines = [f"┌{bar}┐", f"│ {'realizar-b200 monitor':<{width - 1}}│", f"├{bar}┤",
                 f"│ {'throughput  ' + sparkline(list(self.tps), 40) + f'  {self.tps[-1] if self.tps else 0:8.1f} tok/s':<{width - 1}}│",
                 f"│ {'latency ms  p50 %.1f  p95 %.1f  p99 %.1f' % (g('latency_p50_ms'), g('latency_p95_ms'), g('latency_p99_ms')):<{width - 1}}│",
                 f"│ {'requests    total %d  ok %d  failed %d' % (g('total_requests'), g('successful_requests'), g('failed_requests')):<{width - 1}}│",
                 f"│ {'batch       running %s  waiting %s  queue %s' % (g('running', d='-'), g('waiting', d='-'), g('queue_depth', d='-')):<{width - 1}}│",
                 f"│ {'gpu memory  %s MiB used / %s MiB' % (g('gpu_memory_used_mb', d='-'), g('gpu_memory_total_mb', d='-')):<{width - 1}}│",
                 f"└{bar}┘"]
        return "\n".join(lines)


def fetch_metrics(url: str, timeout: float = 2.0) -> dict:
    with urllib.request.urlopen(url.rstrip("/") + "/v1/metrics", timeout=timeout) as r:
        return json.loads(r.read())


def run_monitor(url: str, interval: float = 1.0, once: bool = False, fetch=fetch_metrics, out=print, max_iters: Optional[int] = None) -> int:
    st = MonitorState()
    i = 0
    while True:
        try:
            st.update(fetch(url))
        except Exception as e:
            st.errors += 1
            out(f"(cannot reach {url}: {e})")
            if once:
                return 1
        else:
            out(("\x1b[2J\x1b[H" if not once else "") + st.render())
        i += 1
        if once or (max_iters is not None and i >= max_iters):
            return 0
        time.sleep(interval)
