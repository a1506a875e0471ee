"""Open-loop load generator for the OpenAI-compatible server: Poisson arrivals at a target request
rate with a concurrency cap, streaming chat completions over SSE, and per-request time to first
token / inter-token latency / total latency; reports p50 / p95 / p99 and aggregate tok/s.

Two transports: ``http`` (a running server, aiohttp) and ``inproc`` (the ASGI app driven directly,
no sockets — what the tests and GPU boxes without a listening port use).
Reference parity: the serving benchmarks of the reference's CLI (convoy / saturation / ITL metrics,
src/cli/benchmark.rs:145-355, src/bench/mod.rs ``ItlMetrics``)."""
from __future__ import annotations

import asyncio
import json
import random
import time
from dataclasses import asdict, dataclass, field
from typing import List, Optional

import numpy as np


@dataclass
class LoadConfig:
    requests: int = 200
    rate_per_s: float = 20.0
    max_concurrency: int = 256
    prompt_tokens: int = 64            # approximate: prompts are made of that many short words (or exactly that many characters)
    prompt_tokens_max: int = 0         # > prompt_tokens: every prompt draws its length uniformly from [prompt_tokens, prompt_tokens_max]
    prompt_chars: bool = False         # prompt length counted in characters (byte-level tokenizers: one token per character)
    max_tokens: int = 32
    temperature: float = 0.0
    top_p: float = 1.0
    model: str = "default"
    seed: int = 0
    timeout_s: float = 120.0


@dataclass
class RequestTrace:
    start: float
    first_token: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    end: Optional[float] = None
    tokens: int = 0                       # streamed content events
    generated: Optional[int] = None       # tokens generated according to the server's final usage record
    error: Optional[str] = None

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token is None else self.first_token - self.start


def _pct(xs, q):
    return float(np.percentile(xs, q)) if len(xs) else None


def summarize(traces: List[RequestTrace], wall_s: float) -> dict:
    ok = [t for t in traces if t.error is None and t.end is not None]
    ttft = [1e3 * t.ttft for t in ok if t.ttft is not None]
    itl = [1e3 * d for t in ok for d in np.diff(t.token_times)]
    lat = [1e3 * (t.end - t.start) for t in ok]
    toks = sum(t.generated if t.generated is not None else t.tokens for t in ok)      # generated tokens; events when the server sends no usage
    return {"requests": len(traces), "completed": len(ok), "errors": len(traces) - len(ok), "wall_s": wall_s,
            "req_per_s": len(ok) / wall_s if wall_s else 0.0, "tok_per_s": toks / wall_s if wall_s else 0.0, "tokens": toks, "events": sum(t.tokens for t in ok),
            "ttft_ms": {"p50": _pct(ttft, 50), "p95": _pct(ttft, 95), "p99": _pct(ttft, 99)},
            "itl_ms": {"p50": _pct(itl, 50), "p95": _pct(itl, 95), "p99": _pct(itl, 99)},
            "latency_ms": {"p50": _pct(lat, 50), "p95": _pct(lat, 95), "p99": _pct(lat, 99)}}


def make_prompt(rng: random.Random, n_words: int, chars: bool = False) -> str:
    words = ("the", "of", "and", "model", "token", "cache", "page", "head", "layer", "scale", "block", "warp", "tile", "core", "sum", "max")
    if chars:
        out = ""
        while len(out) < n_words:
            out += rng.choice(words) + " "
        return out[:n_words]
    return " ".join(rng.choice(words) for _ in range(n_words))


def prompt_length(rng: random.Random, cfg: "LoadConfig") -> int:
    return rng.randint(cfg.prompt_tokens, cfg.prompt_tokens_max) if cfg.prompt_tokens_max > cfg.prompt_tokens else cfg.prompt_tokens


def _body(cfg: LoadConfig, prompt: str) -> dict:
    return {"model": cfg.model, "messages": [{"role": "user", "content": prompt}], "max_tokens": cfg.max_tokens, "temperature": cfg.temperature, "top_p": cfg.top_p, "stream": True}


def _consume_sse_line(line: str, tr: RequestTrace) -> bool:
    """Returns True at the end of the stream."""
    if not line.startswith("data:"):
        return False
    data = line[5:].strip()
    if data == "[DONE]":
        return True
    try:
        obj = json.loads(data)
    except ValueError:
        return False
    if "error" in obj:
        tr.error = str(obj["error"])
        return True
    if isinstance(obj.get("usage"), dict) and "completion_tokens" in obj["usage"]:
        tr.generated = int(obj["usage"]["completion_tokens"])          # the server's own count (events can carry several tokens)
    ch = (obj.get("choices") or [{}])[0]
    if (ch.get("delta") or {}).get("content"):
        now = time.perf_counter()
        if tr.first_token is None:
            tr.first_token = now
        tr.token_times.append(now)
        tr.tokens += 1
    return False


async def _one_http(session, url: str, cfg: LoadConfig, prompt: str, tr: RequestTrace) -> None:
    try:
        async with session.post(url + "/v1/chat/completions", json=_body(cfg, prompt)) as resp:
            if resp.status != 200:
                tr.error = f"http {resp.status}"
                return
            async for raw in resp.content:
                if _consume_sse_line(raw.decode("utf-8", "replace").strip(), tr):
                    break
    except Exception as e:                      # noqa: BLE001 - recorded per request
        tr.error = repr(e)
    finally:
        tr.end = time.perf_counter()


async def _one_inproc(app, cfg: LoadConfig, prompt: str, tr: RequestTrace) -> None:
    """Drive the ASGI app directly and parse the SSE body as it is produced."""
    body = json.dumps(_body(cfg, prompt)).encode()
    scope = {"type": "http", "asgi": {"version": "3.0"}, "http_version": "1.1", "method": "POST", "path": "/v1/chat/completions", "raw_path": b"/v1/chat/completions",
             "query_string": b"", "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(body)).encode())], "client": ("127.0.0.1", 0),
             "server": ("127.0.0.1", 80), "scheme": "http", "root_path": ""}
    sent = False
    buf = ""
    done = asyncio.Event()

    async def receive():
        nonlocal sent
        if not sent:
            sent = True
            return {"type": "http.request", "body": body, "more_body": False}
        await done.wait()
        return {"type": "http.disconnect"}

    async def send(msg):
        nonlocal buf
        if msg["type"] == "http.response.start" and msg["status"] != 200:
            tr.error = f"http {msg['status']}"
        elif msg["type"] == "http.response.body":
            buf += msg.get("body", b"").decode("utf-8", "replace")
            while "\n" in buf:
                line, buf = buf.split("\n", 1)
                if _consume_sse_line(line.strip(), tr):
                    done.set()
            if not msg.get("more_body"):
                done.set()
    try:
        await asyncio.wait_for(app(scope, receive, send), cfg.timeout_s)
    except Exception as e:                      # noqa: BLE001
        tr.error = tr.error or repr(e)
    finally:
        tr.end = time.perf_counter()


async def run_load_async(cfg: LoadConfig, url: Optional[str] = None, app=None) -> dict:
    rng = random.Random(cfg.seed)
    sem = asyncio.Semaphore(cfg.max_concurrency)
    traces: List[RequestTrace] = []
    tasks = []
    session = None
    if app is None:
        import aiohttp
        session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=cfg.timeout_s))
    t0 = time.perf_counter()

    async def launch(prompt):
        async with sem:
            tr = RequestTrace(time.perf_counter())
            traces.append(tr)
            if app is not None:
                await _one_inproc(app, cfg, prompt, tr)
            else:
                await _one_http(session, url.rstrip("/"), cfg, prompt, tr)
    try:
        for _ in range(cfg.requests):
            tasks.append(asyncio.create_task(launch(make_prompt(rng, prompt_length(rng, cfg), cfg.prompt_chars))))
            if cfg.rate_per_s > 0:
                await asyncio.sleep(rng.expovariate(cfg.rate_per_s))        # Poisson arrivals
        await asyncio.gather(*tasks)
    finally:
        if session is not None:
            await session.close()
    out = summarize(traces, time.perf_counter() - t0)
    out["config"] = asdict(cfg)
    return out


def run_load(cfg: LoadConfig, url: Optional[str] = None, app=None) -> dict:
    return asyncio.run(run_load_async(cfg, url, app))
