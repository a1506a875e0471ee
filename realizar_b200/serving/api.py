"""HTTP API: OpenAI-compatible chat / completions / embeddings / models, native generate /
tokenize / batch / stream routes, health, Prometheus and JSON metrics, dispatch metrics, audit
trail, GPU status / warm-up, log-probabilities and perplexity.

Route set and JSON schemas follow the reference router (src/api/router.rs:57-135;
chat request / response / chunk types src/api/mod_create_demo.rs:62-330; SSE sequence
role -> content deltas -> finish -> ``[DONE]`` src/api/openai_handlers.rs:179-275; native types
src/api/types.rs).  A full queue answers 503, malformed bodies 422 with a sanitised message,
unknown paths a JSON 404.
"""
from __future__ import annotations

import asyncio
import json
import math
import threading
import time
import uuid
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Header, HTTPException, Request as HttpRequest
from fastapi.exceptions import RequestValidationError
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from pydantic import BaseModel, Field

from .. import __version__
from ..runtime.scheduler import FinishReason, QueueFull, Request, ServingEngine
from .chat_template import ChatMessage, ChatTemplate, RawTemplate, auto_detect_template
from .metrics import DispatchMetrics, MetricsCollector
from .tokenizer import StreamDecoder

KEEP_ALIVE_SECONDS = 15.0


# ------------------------------------------------------------------ schemas ---------------
class ChatMessageIn(BaseModel):
    role: str
    content: str = ""
    name: Optional[str] = None


class ChatCompletionRequest(BaseModel):
    model: str = "default"
    messages: List[ChatMessageIn]
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    n: int = 1
    stream: bool = False
    stop: Optional[List[str]] = None
    user: Optional[str] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[Dict[str, float]] = None
    response_format: Optional[Dict[str, Any]] = None       # {"type": "json_object"} | {"type": "json_schema", "json_schema": {...}}
    grammar: Optional[str] = None                           # GBNF text


class CompletionRequest(BaseModel):
    model: str = "default"
    prompt: str
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    stop: Optional[List[str]] = None
    stream: bool = False
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[Dict[str, float]] = None
    response_format: Optional[Dict[str, Any]] = None
    grammar: Optional[str] = None


class GenerateRequest(BaseModel):
    prompt: str
    max_tokens: int = 50
    temperature: float = 1.0
    strategy: str = "greedy"
    top_k: int = 50
    top_p: float = 0.9
    seed: Optional[int] = None
    model_id: Optional[str] = None


class TokenizeRequest(BaseModel):
    text: str
    model_id: Optional[str] = None


class BatchTokenizeRequest(BaseModel):
    texts: List[str]


class BatchGenerateRequest(BaseModel):
    prompts: List[str]
    max_tokens: int = 50
    temperature: float = 1.0
    strategy: str = "greedy"
    top_k: int = 50
    top_p: float = 0.9


class EmbeddingRequest(BaseModel):
    model: str = "default"
    input: Any


class LogprobsRequest(BaseModel):
    prompt: str
    top_logprobs: int = 5


@dataclass
class AppState:
    serving: Optional[ServingEngine]
    tokenizer: Any
    template: ChatTemplate = field(default_factory=RawTemplate)
    model_name: str = "default"
    eos_token_id: Optional[int] = None
    metrics: MetricsCollector = field(default_factory=MetricsCollector)
    dispatch: DispatchMetrics = field(default_factory=DispatchMetrics)
    audit: Dict[str, dict] = field(default_factory=dict)
    compute_mode: str = "gpu"
    scorer: Any = None                  # object with logprobs(ids) / embed(ids) (runtime.scorer.EngineScorer for GPU engines)
    vocab_strings: Optional[List[str]] = None       # text of every token id, built on the first grammar-constrained request
    context_length: int = 4096
    classical: Any = None               # optional ClassicalServeState behind /v1/predict, /v1/explain
    fanouts: Dict[Any, Any] = field(default_factory=dict)             # event loop -> TokenFanout (engine thread -> stream queues)
    route_latency: Dict[str, Any] = field(default_factory=dict)      # path -> LatencyHistogram of whole HTTP requests
    spans: Any = field(default_factory=lambda: deque(maxlen=256))    # finished request spans, newest last (GET /v1/traces)

    @classmethod
    def demo(cls) -> "AppState":
        """A self-contained state with a fake engine and a byte tokenizer (tests, smoke runs)."""
        from ..runtime.scheduler import FakeEngine
        from ..runtime.scorer import EngineScorer
        from .tokenizer import ByteTokenizer
        serving = ServingEngine(FakeEngine(vocab=256)).start()
        return cls(serving, ByteTokenizer(256), RawTemplate(), "demo", None, compute_mode="cpu", scorer=EngineScorer(serving))


class TokenFanout:
    """Delivery of engine-thread events (tokens, request ends) to the per-stream asyncio queues with ONE event-loop wake-up per
    burst instead of one per token: the engine thread appends to a list and schedules a drain only when none is pending, the
    drain (on the loop thread) moves everything posted so far into the queues.  At 256 streams a decode step posts 256 tokens;
    256 ``call_soon_threadsafe`` calls mean 256 writes to the loop's wake-up pipe and as many lock hand-overs."""

    def __init__(self, loop: "asyncio.AbstractEventLoop"):
        self.loop = loop
        self._items: List[tuple] = []
        self._lock = threading.Lock()
        self._scheduled = False

    def post(self, q: "asyncio.Queue", item) -> None:
        with self._lock:
            self._items.append((q, item))
            if self._scheduled:
                return
            self._scheduled = True
        self.loop.call_soon_threadsafe(self._drain)

    def _drain(self) -> None:
        with self._lock:
            items, self._items = self._items, []
            self._scheduled = False
        for q, item in items:
            q.put_nowait(item)


def _finish_reason(r: Request) -> str:
    return "stop" if r.finish_reason == FinishReason.STOP else "length"


def create_app(state: AppState) -> FastAPI:
    app = FastAPI(title="realizar-b200", version=__version__)
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    app.state.rlz = state

    @app.middleware("http")
    async def _trace(request: HttpRequest, call_next):
        """W3C trace context in and out (``traceparent``), one span and one latency observation per HTTP request
        (role of the reference's trace-context / span / latency-histogram types, src/observability/mod.rs:47-421)."""
        from ..utils.observability import LatencyHistogram, Span, TraceContext
        ctx = TraceContext.from_traceparent(request.headers.get("traceparent", "")) or TraceContext.new()
        span = Span(f"{request.method} {request.url.path}", ctx)
        try:
            resp = await call_next(request)
        except Exception:
            state.spans.append(span.end(ok=False))
            raise
        span.set("http.status_code", resp.status_code).end(ok=resp.status_code < 500)
        state.spans.append(span)
        hist = state.route_latency.get(request.url.path)
        if hist is None and len(state.route_latency) < 64:           # unknown paths (404 probes) must not grow the table without bound
            hist = state.route_latency[request.url.path] = LatencyHistogram()
        if hist is not None:
            hist.observe(span.duration_ms)
        resp.headers["traceparent"] = ctx.to_traceparent()
        return resp

    @app.get("/v1/traces")
    async def traces(limit: int = 50):
        return {"spans": [sp.to_otel() for sp in list(state.spans)[-max(1, min(limit, 256)):]]}

    @app.exception_handler(RequestValidationError)
    async def _validation(_req, exc: RequestValidationError):
        msgs = "; ".join(f"{'.'.join(str(x) for x in e.get('loc', [])[1:])}: {e.get('msg', '')}" for e in exc.errors())
        return JSONResponse({"error": f"invalid request: {msgs}"[:500]}, status_code=422)

    @app.exception_handler(404)
    async def _not_found(_req, _exc):
        return JSONResponse({"error": "not found"}, status_code=404)

    # -- helpers ---------------------------------------------------------------------------------
    def encode(text: str) -> List[int]:
        ids = state.tokenizer.encode(text)
        if not ids:
            raise HTTPException(400, "prompt is empty after tokenisation")
        if len(ids) >= state.context_length:                      # context-window manager: keep the most recent tokens
            ids = ids[-(state.context_length - 1):]
        return ids

    def stop_ids() -> List[int]:
        return [state.eos_token_id] if state.eos_token_id is not None else []

    def vocab_strings() -> List[str]:
        """Text of every token id (grammar masks test tokens as strings); built once per server."""
        if state.vocab_strings is None:
            tok = state.tokenizer
            n = getattr(tok, "vocab_size", None) or len(getattr(tok, "vocab", []))
            state.vocab_strings = [tok.decode([i]) for i in range(int(n))]
        return state.vocab_strings

    def controls_of(req) -> dict:
        """Request-level sampling controls of an OpenAI-style body as ``Request`` fields: penalties, logit_bias, a grammar /
        JSON-schema token mask and a stop-string check (the generation ends when a stop string appears in the decoded text)."""
        extra: Dict[str, Any] = {}
        for k in ("presence_penalty", "frequency_penalty"):
            if getattr(req, k, 0.0):
                extra[k] = float(getattr(req, k))
        if getattr(req, "repetition_penalty", 1.0) not in (None, 1.0):
            extra["repetition_penalty"] = float(req.repetition_penalty)
        if getattr(req, "min_p", None):
            extra["min_p"] = float(req.min_p)
        if getattr(req, "logit_bias", None):
            try:
                extra["logit_bias"] = {int(k): float(v) for k, v in req.logit_bias.items()}
            except ValueError:
                raise HTTPException(400, "logit_bias keys must be token ids")
        gtext, rf = getattr(req, "grammar", None), getattr(req, "response_format", None)
        if gtext or (rf and rf.get("type") in ("json_object", "json_schema")):
            from .grammar import Grammar, GrammarTokenMasker, grammar_from_json_schema
            try:
                if gtext:
                    g = Grammar.from_gbnf(gtext)
                else:
                    schema = (rf.get("json_schema") or {}).get("schema", rf.get("json_schema")) if rf.get("type") == "json_schema" else {"type": "object"}
                    g = grammar_from_json_schema(schema or {"type": "object"})
            except Exception as e:
                raise HTTPException(400, f"invalid grammar: {e}")
            extra["token_masker"] = GrammarTokenMasker(g, vocab_strings(), state.eos_token_id)
        stops = [s for s in (getattr(req, "stop", None) or []) if s]
        if stops:
            def stop_check(r: Request, stops=stops) -> bool:
                text = state.tokenizer.decode(r.output[-64:])
                return any(s in text for s in stops)
            extra["stop_check"] = stop_check
        return extra

    def submit(prompt_ids, max_tokens, temperature, top_k, top_p, on_token=None, on_finish=None, extra: Optional[dict] = None) -> Request:
        if state.serving is None:
            raise HTTPException(503, "no model loaded")
        r = Request(prompt_ids, max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p, stop_token_ids=stop_ids(),
                    on_token=on_token, on_finish=on_finish, **(extra or {}))
        try:
            state.serving.submit(r)
        except QueueFull:
            state.metrics.record_failure()
            raise HTTPException(503, "server is at capacity, retry later")
        except RuntimeError as e:
            state.metrics.record_failure()
            raise HTTPException(503, str(e))
        return r

    async def run_blocking(prompt_ids, max_tokens, temperature, top_k, top_p, extra: Optional[dict] = None) -> Request:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        r = submit(prompt_ids, max_tokens, temperature, top_k, top_p,
                   on_finish=lambda rq: loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(rq)), extra=extra)
        await fut
        record(r)
        if r.finish_reason == FinishReason.ERROR:
            raise HTTPException(500, r.error or "generation failed")
        return r

    def record(r: Request) -> None:
        state.dispatch.record(state.compute_mode, (r.finish_time or time.monotonic()) - r.arrival)
        if r.finish_reason == FinishReason.ERROR:
            state.metrics.record_failure()
        else:
            state.metrics.record_success(len(r.output), (r.finish_time or time.monotonic()) - r.arrival, r.ttft, r.token_times)

    def text_of(r: Request) -> str:
        toks = r.output[:-1] if r.finish_reason == FinishReason.STOP and r.output and r.output[-1] in stop_ids() else r.output
        return state.tokenizer.decode(toks)

    def apply_stops(text: str, stops: Optional[List[str]]) -> str:
        for s in stops or []:
            i = text.find(s)
            if i >= 0:
                text = text[:i]
        return text

    def chat_params(req) -> tuple:
        t = 0.7 if req.temperature is None else req.temperature
        k = getattr(req, "top_k", None)
        return (req.max_tokens or 256, t, 1 if t == 0 else (40 if k is None else int(k)), 1.0 if req.top_p is None else req.top_p)

    def audit(rid: str, kind: str, prompt_tokens: int, completion_tokens: int, latency: float) -> None:
        state.audit[rid] = {"request_id": rid, "endpoint": kind, "model": state.model_name, "prompt_tokens": prompt_tokens,
                            "completion_tokens": completion_tokens, "latency_ms": 1e3 * latency, "timestamp": time.time()}
        if len(state.audit) > 10000:
            state.audit.pop(next(iter(state.audit)))

    def trace_block(level: Optional[str], r: Request) -> dict:
        if level not in ("brick", "step", "layer"):
            return {}
        total = 1e6 * ((r.finish_time or time.monotonic()) - r.arrival)
        return {f"{level}_trace": {"level": level, "total_time_us": total, "ttft_us": 1e6 * (r.ttft or 0.0),
                                   "operations": [{"name": "prefill", "time_us": 1e6 * (r.ttft or 0.0)}, {"name": "decode", "time_us": total - 1e6 * (r.ttft or 0.0)}]}}

    def sse_stream(r_holder: dict, first_chunk: Optional[dict], make_chunk, done_chunk):
        """Server-sent events fed by the engine thread through an asyncio queue."""
        async def gen():
            loop = asyncio.get_running_loop()
            fan = state.fanouts.get(loop)
            if fan is None:
                fan = state.fanouts[loop] = TokenFanout(loop)
            q: asyncio.Queue = asyncio.Queue()
            dec = StreamDecoder(state.tokenizer)
            stops = set(stop_ids())
            r = submit(*r_holder["args"], on_token=lambda t: fan.post(q, ("tok", t)),
                       on_finish=lambda rq: fan.post(q, ("end", rq)), extra=r_holder.get("extra"))
            stop_strs = r_holder.get("stops") or []
            held = ""                                        # text not yet sent: a stop string may still be forming at its end
            if first_chunk is not None:
                yield f"data: {json.dumps(first_chunk)}\n\n"
            try:
                while True:
                    try:
                        kind, val = await asyncio.wait_for(q.get(), KEEP_ALIVE_SECONDS)
                    except asyncio.TimeoutError:
                        yield ": keep-alive\n\n"
                        continue
                    if kind == "tok":
                        # tokens that piled up while this stream waited for the loop go out as ONE event: under load the
                        # per-event cost (JSON, HTTP framing, a socket write) is what limits the server, not the tokens
                        text, pending_end = ("" if val in stops else dec.push(val)), None
                        while not q.empty():
                            k2, v2 = q.get_nowait()
                            if k2 != "tok":
                                pending_end = (k2, v2)
                                break
                            if v2 not in stops:
                                text += dec.push(v2)
                                val = v2
                        if pending_end is not None:
                            q.put_nowait(pending_end)          # (nothing can follow a request's end: order is kept)
                        if text and stop_strs:
                            held += text
                            cut = min((held.find(s_) for s_ in stop_strs if s_ in held), default=-1)
                            if cut >= 0:                     # the stop string itself is never sent
                                text, held = held[:cut], ""
                                stop_strs = []
                                r.cancelled = r.finish_reason is None
                            else:
                                keep = max(len(s_) for s_ in stop_strs) - 1
                                text, held = (held[:-keep], held[-keep:]) if keep > 0 and len(held) > keep else ("", held) if keep > 0 else (held, "")
                        if text:
                            yield f"data: {json.dumps(make_chunk(val, text))}\n\n"
                    else:
                        record(val)
                        if val.finish_reason == FinishReason.ERROR:
                            yield f"data: {json.dumps({'error': val.error or 'generation failed'})}\n\n"
                        else:
                            tail = dec.flush()
                            if r_holder.get("stops"):
                                tail = apply_stops(held + tail, r_holder.get("stops")) if stop_strs else ""
                            if tail:
                                yield f"data: {json.dumps(make_chunk(-1, tail))}\n\n"
                            yield f"data: {json.dumps(done_chunk(val))}\n\n"
                        yield "data: [DONE]\n\n"
                        return
            finally:
                r.cancelled = r.finish_reason is None          # client went away: stop generating
        return StreamingResponse(gen(), media_type="text/event-stream")

    # -- health / metrics --------------------------------------------------------------------------
    @app.get("/health")
    async def health():
        h = state.serving.health if state.serving is not None else "no_model"
        body = {"status": "healthy" if h == "ok" else h, "version": __version__, "compute_mode": state.compute_mode}
        return JSONResponse(body, status_code=200 if h in ("ok", "no_model") else 503)

    def refresh_gauges():
        if state.serving is not None:
            m = state.serving.metrics()
            for k in ("queue_depth", "running", "kv_page_utilization", "avg_step_ms"):
                state.metrics.set_gauge(k, m.get(k, 0))

    @app.get("/metrics")
    async def metrics():
        refresh_gauges()
        return PlainTextResponse(state.metrics.prometheus(), media_type="text/plain; version=0.0.4")

    @app.get("/v1/metrics")
    async def metrics_json():
        refresh_gauges()
        snap = state.metrics.snapshot()
        if state.serving is not None:
            snap["scheduler"] = state.serving.metrics()
        snap["http_latency_ms"] = {path: {"count": h.total, "mean": round(h.mean_ms, 3), "p50_le": h.percentile(50), "p99_le": h.percentile(99)}
                                   for path, h in state.route_latency.items()}
        return snap

    @app.get("/metrics/dispatch")
    async def dispatch(format: str = "json"):
        return PlainTextResponse(state.dispatch.prometheus()) if format == "prometheus" else state.dispatch.to_dict()

    @app.post("/metrics/dispatch/reset")
    async def dispatch_reset():
        state.dispatch.reset()
        return {"status": "reset"}

    # -- models ------------------------------------------------------------------------------------
    @app.get("/models")
    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": state.model_name, "object": "model", "created": int(state.metrics.start), "owned_by": "realizar-b200"}]}

    @app.get("/realize/model")
    async def realize_model():
        return {"model": state.model_name, "context_length": state.context_length, "template": state.template.format, "compute_mode": state.compute_mode}

    @app.post("/realize/reload")
    async def realize_reload():
        raise HTTPException(501, "hot reload needs the process to be started with a model registry (see `realizar-b200 serve --help`)")

    # -- tokenize / native generate ----------------------------------------------------------------
    @app.post("/tokenize")
    async def tokenize(req: TokenizeRequest):
        ids = state.tokenizer.encode(req.text)
        return {"token_ids": ids, "num_tokens": len(ids)}

    @app.post("/batch/tokenize")
    async def batch_tokenize(req: BatchTokenizeRequest):
        out = [state.tokenizer.encode(t) for t in req.texts]
        return {"results": [{"token_ids": ids, "num_tokens": len(ids)} for ids in out]}

    def native_params(req) -> tuple:
        greedy = req.strategy == "greedy" or req.temperature == 0
        return (req.max_tokens, 0.0 if greedy else req.temperature, 1 if greedy else (req.top_k if req.strategy in ("top_k", "top_p") else 0),
                req.top_p if req.strategy == "top_p" else 1.0)

    @app.post("/generate")
    @app.post("/realize/generate")
    async def generate(req: GenerateRequest):
        if req.strategy not in ("greedy", "top_k", "top_p", "sample"):
            raise HTTPException(400, f"unknown strategy '{req.strategy}'")
        ids = encode(req.prompt)
        r = await run_blocking(ids, *native_params(req))
        return {"token_ids": r.output, "text": text_of(r), "num_generated": len(r.output)}

    @app.post("/batch/generate")
    @app.post("/realize/batch")
    async def batch_generate(req: BatchGenerateRequest):
        if not req.prompts:
            raise HTTPException(400, "prompts is empty")
        rs = await asyncio.gather(*[run_blocking(encode(p), *native_params(req)) for p in req.prompts])
        return {"results": [{"token_ids": r.output, "text": text_of(r), "num_generated": len(r.output)} for r in rs]}

    @app.post("/stream/generate")
    async def stream_generate(req: GenerateRequest):
        ids = encode(req.prompt)
        holder = {"args": (ids, *native_params(req))}
        return sse_stream(holder, None, lambda tid, text: {"token_id": tid, "text": text}, lambda r: {"num_generated": len(r.output)})

    # -- OpenAI ------------------------------------------------------------------------------------
    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatCompletionRequest, x_trace_level: Optional[str] = Header(default=None)):
        if not req.messages:
            raise HTTPException(400, "messages is empty")
        prompt = state.template.format_conversation([ChatMessage(m.role, m.content, m.name) for m in req.messages])
        ids = encode(prompt)
        rid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        params = chat_params(req)
        if req.stream:
            base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": req.model}
            first = {**base, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}
            return sse_stream({"args": (ids, *params), "extra": controls_of(req), "stops": req.stop}, first,
                              lambda _tid, text: {**base, "choices": [{"index": 0, "delta": {"content": text}, "finish_reason": None}]},
                              lambda r: {**base, "choices": [{"index": 0, "delta": {}, "finish_reason": _finish_reason(r)}],
                                         "usage": {"prompt_tokens": len(ids), "completion_tokens": len(r.output), "total_tokens": len(ids) + len(r.output)}})
        r = await run_blocking(ids, *params, extra=controls_of(req))
        text = apply_stops(text_of(r), req.stop)
        audit(rid, "chat.completions", len(ids), len(r.output), (r.finish_time or time.monotonic()) - r.arrival)
        return {"id": rid, "object": "chat.completion", "created": created, "model": req.model,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": _finish_reason(r)}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(r.output), "total_tokens": len(ids) + len(r.output)},
                **trace_block(x_trace_level, r)}

    @app.post("/v1/chat/completions/stream")
    async def chat_completions_stream(req: ChatCompletionRequest):
        req.stream = True
        return await chat_completions(req, None)

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest):
        ids = encode(req.prompt)
        rid, created = f"cmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        params = chat_params(req)
        if req.stream:
            base = {"id": rid, "object": "text_completion", "created": created, "model": req.model}
            return sse_stream({"args": (ids, *params), "extra": controls_of(req), "stops": req.stop}, None,
                              lambda _tid, text: {**base, "choices": [{"index": 0, "text": text, "finish_reason": None}]},
                              lambda r: {**base, "choices": [{"index": 0, "text": "", "finish_reason": _finish_reason(r)}]})
        r = await run_blocking(ids, *params, extra=controls_of(req))
        audit(rid, "completions", len(ids), len(r.output), (r.finish_time or time.monotonic()) - r.arrival)
        return {"id": rid, "object": "text_completion", "created": created, "model": req.model,
                "choices": [{"index": 0, "text": apply_stops(text_of(r), req.stop), "finish_reason": _finish_reason(r)}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(r.output), "total_tokens": len(ids) + len(r.output)}}

    @app.post("/v1/batch/completions")
    async def batch_completions(body: Dict[str, Any]):
        prompts = body.get("prompts") or []
        if not prompts:
            raise HTTPException(400, "prompts is empty")
        t = body.get("temperature", 0.7)
        rs = await asyncio.gather(*[run_blocking(encode(p), body.get("max_tokens", 256), t, 1 if t == 0 else 40, body.get("top_p", 1.0)) for p in prompts])
        return {"object": "list", "data": [{"index": i, "text": text_of(r), "finish_reason": _finish_reason(r)} for i, r in enumerate(rs)]}

    @app.post("/v1/embeddings")
    @app.post("/realize/embed")
    async def embeddings(req: EmbeddingRequest):
        texts = req.input if isinstance(req.input, list) else [req.input]
        if state.scorer is None or not hasattr(state.scorer, "embed"):
            raise HTTPException(501, "this server was started without an embedding-capable model")
        data = [{"object": "embedding", "index": i, "embedding": [float(v) for v in state.scorer.embed(state.tokenizer.encode(str(t)))]} for i, t in enumerate(texts)]
        return {"object": "list", "data": data, "model": req.model, "usage": {"prompt_tokens": sum(len(state.tokenizer.encode(str(t))) for t in texts)}}

    @app.post("/v1/logprobs")
    async def logprobs(req: LogprobsRequest):
        if state.scorer is None:
            raise HTTPException(501, "this server was started without a scoring model")
        ids = encode(req.prompt)
        lp = state.scorer.logprobs(ids)                      # [T-1] log p(token_t | prefix)
        return {"tokens": ids, "token_logprobs": [None] + [float(x) for x in lp]}

    @app.post("/v1/perplexity")
    async def perplexity(body: Dict[str, Any]):
        if state.scorer is None:
            raise HTTPException(501, "this server was started without a scoring model")
        ids = encode(str(body.get("text", "")))
        if len(ids) < 2:
            raise HTTPException(400, "need at least two tokens")
        lp = state.scorer.logprobs(ids)
        nll = -float(sum(lp)) / len(lp)
        return {"perplexity": math.exp(nll), "nll": nll, "num_tokens": len(ids)}

    @app.get("/v1/audit/{request_id}")
    async def audit_get(request_id: str):
        if state.classical is not None:
            rec = state.classical.sink.get(request_id)
            if rec is not None:
                return json.loads(rec.to_json())
        if request_id not in state.audit:
            raise HTTPException(404, f"audit record '{request_id}' not found")
        return state.audit[request_id]

    def _classical(body: Dict[str, Any], explain: bool):
        if state.classical is None:
            raise HTTPException(501, "no classical model loaded (start with `serve --classical <model.apr>`)")
        feats = body.get("features")
        if not isinstance(feats, list) or not feats:
            raise HTTPException(400, "features must be a non-empty list of numbers")
        try:
            return state.classical.predict(feats, explain=explain or bool(body.get("explain")), client=body.get("user"))
        except ValueError as e:
            raise HTTPException(400, str(e))

    @app.post("/v1/predict")
    async def predict(body: Dict[str, Any]):
        return _classical(body, False)

    @app.post("/v1/explain")
    async def explain(body: Dict[str, Any]):
        return _classical(body, True)

    # -- GPU ---------------------------------------------------------------------------------------
    @app.get("/v1/gpu/status")
    async def gpu_status():
        try:
            import torch
            if not torch.cuda.is_available():
                return {"available": False}
            free, total = torch.cuda.mem_get_info()
            return {"available": True, "device": torch.cuda.get_device_name(0), "memory_free": free, "memory_total": total,
                    "engine": state.serving.metrics() if state.serving else None}
        except Exception as e:
            return {"available": False, "error": str(e)}

    @app.post("/v1/gpu/warmup")
    async def gpu_warmup():
        if state.serving is None:
            raise HTTPException(503, "no model loaded")
        t0 = time.monotonic()
        r = await run_blocking(encode("warm up"), 4, 0.0, 1, 1.0)
        return {"status": "ok", "tokens": len(r.output), "seconds": time.monotonic() - t0}

    @app.post("/v1/gpu/reset")
    async def gpu_reset():
        """Bring a server back whose engine loop stopped after a failed step (health "unhealthy"): the engine is probed and
        reset in place; 503 when the device context is lost and the process has to be restarted."""
        if state.serving is None:
            raise HTTPException(503, "no model loaded")
        ok = await asyncio.get_running_loop().run_in_executor(None, state.serving.recover)
        if not ok:
            raise HTTPException(503, f"engine cannot be recovered in place: {state.serving.last_error}")
        return {"status": "ok", "health": state.serving.health}

    return app


def serve(state: AppState, host: str = "127.0.0.1", port: int = 8080, log_level: str = "warning") -> None:
    import uvicorn
    uvicorn.run(create_app(state), host=host, port=port, log_level=log_level)
