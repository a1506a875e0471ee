"""Scheduler, serving loop (fake engine), tokenizers, chat templates, samplers, metrics and the HTTP API."""
import json
import threading
import time

import numpy as np
import pytest

from realizar_b200.runtime.scheduler import (FakeEngine, FinishReason, QueueFull, Request, RequestState, Scheduler, SchedulerConfig,
                                             ServingEngine)
from realizar_b200.serving import sampling as S
from realizar_b200.serving.chat_template import (ChatMessage, ChatTemplateError, HuggingFaceTemplate, auto_detect_template,
                                                 detect_format_from_name, format_messages)
from realizar_b200.serving.metrics import DispatchMetrics, LatencyHistogram, MetricsCollector
from realizar_b200.serving.tokenizer import BPETokenizer, SentencePieceTokenizer, StreamDecoder, bytes_to_unicode


# ---------------------------------------------------------------------------- scheduler --------
def test_scheduler_admission_decode_and_recycling():
    s = Scheduler(SchedulerConfig(max_batch=2, max_seq_len=64, token_budget=64, prefill_chunk=8))
    rs = [s.add_request(Request([1, 2, 3] * 4, max_tokens=3)) for _ in range(3)]
    d = s.schedule()
    assert len(d.admitted) == 2 and len(d.prefill) == 1 and d.prefill[0][1:] == (0, 8)      # one chunked prefill per iteration
    s.on_prefill_done(d.prefill[0][0], 8, None)
    d = s.schedule()
    r0 = d.prefill[0][0]
    assert d.prefill[0][1:] == (8, 12)
    s.on_prefill_done(r0, 12, 42)
    assert r0.state == RequestState.RUNNING and r0.output == [42] and r0.ttft is not None
    d = s.schedule()
    assert r0 in d.decode
    s.on_token(r0, 7); s.on_token(r0, 8)
    assert r0.state == RequestState.FINISHED and r0.finish_reason == FinishReason.LENGTH
    d = s.schedule()
    assert rs[2] in d.admitted                                                            # freed slot is recycled
    with pytest.raises(ValueError):
        s.add_request(Request(list(range(100))))


def test_scheduler_priority_aging_preemption_and_queue_bound():
    s = Scheduler(SchedulerConfig(max_batch=1, max_seq_len=64, max_waiting=2), total_pages=4)
    low = s.add_request(Request([1] * 8, max_tokens=40, priority=0))
    s.schedule()
    assert low.state == RequestState.PREFILL
    high = s.add_request(Request([2] * 8, max_tokens=40, priority=5))
    s.free_slots.append(1)                                  # a second slot, but the KV pages are exhausted
    d = s.schedule()
    assert low in d.preempted and high in d.admitted and low.state == RequestState.PREEMPTED
    s.add_request(Request([3], priority=0))
    with pytest.raises(QueueFull):
        s.add_request(Request([4])); s.add_request(Request([5]))
    old = Request([9], priority=0); old.arrival -= 100
    new = Request([9], priority=3)
    s2 = Scheduler(SchedulerConfig(max_batch=1, aging_seconds=5.0))
    s2.add_request(new); s2.add_request(old)
    assert s2.schedule().admitted == [old]                  # aging beats the static priority


def test_serving_engine_continuous_batching_with_fake_engine():
    eng = FakeEngine(max_batch=2, vocab=50)
    srv = ServingEngine(eng, SchedulerConfig(max_batch=2, max_seq_len=256)).start()
    try:
        got = []
        rs = [srv.generate([i, i + 1], max_tokens=5, stop_token_ids=[49]) for i in (1, 10)]
        assert rs[0].output == [3, 4, 5, 6, 7] and rs[1].output == [12, 13, 14, 15, 16]
        done = threading.Event()
        r = Request([45], max_tokens=20, stop_token_ids=[49], on_token=got.append, on_finish=lambda _: done.set())
        srv.submit(r); assert done.wait(5)
        assert got == [46, 47, 48, 49] and r.finish_reason == FinishReason.STOP
        evs = [threading.Event() for _ in range(5)]
        many = [Request([i], max_tokens=4, on_finish=lambda _r, e=e: e.set()) for i, e in enumerate(evs)]
        for m in many:
            srv.submit(m)
        assert all(e.wait(5) for e in evs)
        assert any(c[0] == "feed" and len(c[1]) == 2 for c in eng.calls)          # two sequences shared a decode step
        assert not eng.open                                                       # every slot was closed again
        assert srv.metrics()["finished"] == 8
    finally:
        srv.stop()


def test_serving_engine_failure_latches_unhealthy_and_client_abort():
    srv = ServingEngine(FakeEngine(max_batch=1, fail_after=2)).start()
    try:
        r = srv.generate([1], max_tokens=50, timeout=5)
        assert r.finish_reason == FinishReason.ERROR and "injected" in r.error
        assert srv.health == "unhealthy"
        with pytest.raises(RuntimeError):
            srv.submit(Request([1]))
    finally:
        srv.stop()
    srv = ServingEngine(FakeEngine(max_batch=1)).start()
    try:
        done = threading.Event()
        def boom(_t):
            raise ConnectionError("client went away")
        r = Request([1], max_tokens=50, on_token=boom, on_finish=lambda _: done.set())
        srv.submit(r); assert done.wait(5)
        assert r.finish_reason == FinishReason.ABORT and len(r.output) == 1
    finally:
        srv.stop()


# ---------------------------------------------------------------------------- text -------------
def test_tokenizers_round_trip_and_specials():
    b2u = bytes_to_unicode()
    vocab = [b2u[i] for i in range(256)] + ["Ġhello", "Ġworld", "he", "llo", "<|im_end|>"]
    t = BPETokenizer(vocab, eos_token_id=260)
    text = "hello world<|im_end|> héllo\n"
    ids = t.encode(text)
    assert t.decode(ids) == text and 260 in ids and ids[:2] == [258, 259]
    merged = BPETokenizer(vocab + ["Ġw", "Ġwo"], merges=["Ġ w", "Ġw o"])
    assert merged.decode(merged.encode(" wow")) == " wow" and merged.encode(" wo")[0] == merged.vocab.index["Ġwo"]
    sd = StreamDecoder(t)
    assert "".join(sd.push(i) for i in t.encode("é€")) + sd.flush() == "é€"
    sp = SentencePieceTokenizer(["<unk>", "<s>", "</s>", "▁he", "llo", "▁hello", "▁world"] + [f"<0x{i:02X}>" for i in range(256)],
                                [0, 0, 0, -2, -2, -1, -1.5] + [-10] * 256, bos_token_id=1)
    ids = sp.encode("hello world é")
    assert ids[:3] == [1, 5, 6] and sp.decode(ids[1:]) == "hello world é"


def test_chat_templates_and_detection():
    msgs = [ChatMessage.system("Be brief."), ChatMessage.user("Hi <|im_end|>")]
    out = format_messages(msgs, "Qwen2-0.5B-Instruct")
    assert out.startswith("<|im_start|>system\nBe brief.<|im_end|>\n") and out.endswith("<|im_start|>assistant\n")
    assert "<|im_end|>\n<|im_start|>assistant" in out and "Hi <|im_end|>" not in out          # injection neutralised
    assert detect_format_from_name("TinyLlama-1.1B") == "zephyr" and detect_format_from_name("Mixtral-8x7B") == "mistral"
    assert detect_format_from_name("phi-2") == "phi" and detect_format_from_name("unknown") == "raw"
    assert format_messages(msgs, "phi-2").endswith("Output:")
    assert "<<SYS>>\nBe brief.\n<</SYS>>" in format_messages(msgs, "llama-2-7b-chat")
    assert format_messages(msgs, "qwen3-8b").endswith("<think>\n</think>\n")
    assert "[INST] Hi" in format_messages(msgs, "mistral-7b") and "Be brief" not in format_messages(msgs, "mistral-7b")
    hf = HuggingFaceTemplate("{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}{% if add_generation_prompt %}[assistant]{% endif %}")
    assert hf.format_conversation(msgs).endswith("[assistant]")
    with pytest.raises(ChatTemplateError):
        HuggingFaceTemplate("{% for %}")
    with pytest.raises(ChatTemplateError):
        auto_detect_template("qwen").format_conversation([ChatMessage.user("x" * 200_000)])


# ---------------------------------------------------------------------------- sampling ---------
def test_truncation_samplers():
    logits = np.log(np.array([0.5, 0.25, 0.15, 0.07, 0.03]))
    assert np.isfinite(S.top_k_filter(logits, 2)).sum() == 2
    assert np.isfinite(S.top_p_filter(logits, 0.7)).sum() == 2 and np.isfinite(S.top_p_filter(logits, 0.76)).sum() == 3
    assert np.isfinite(S.min_p_filter(logits, 0.2)).sum() == 3
    assert np.isfinite(S.typical_filter(logits, 0.5)).sum() >= 1 and np.isfinite(S.tfs_filter(logits, 0.5)).sum() < 5
    assert np.isfinite(S.eta_filter(logits, epsilon_cutoff=0.1)).sum() == 3
    rng = np.random.default_rng(0)
    x = S.xtc_filter(logits, 1.0, 0.2, rng)
    assert not np.isfinite(x[0]) and np.isfinite(x[1])                                  # top choice excluded, least likely above threshold kept
    pen = S.apply_repetition_penalties(np.array([2.0, -2.0, 1.0]), [0, 1, 0], 2.0, 0.5, 0.25)
    assert np.allclose(pen, [1.0 - 0.5 - 0.5, -4.0 - 0.5 - 0.25, 1.0])
    assert S.dynamic_temperature(np.zeros(10), 1.0, 0.5) == pytest.approx(1.5) and S.dynamic_temperature(logits, 1.0, 0.0) == 1.0
    dry = S.dry_penalty(np.zeros(10), [1, 2, 3, 4, 1, 2, 3], 1.0, 2.0, 2)
    assert dry[4] == pytest.approx(-2.0) and np.count_nonzero(dry) == 1                 # "1 2 3" repeated -> 4 is penalised
    g = S.cfg_combine(logits, np.zeros(5), 1.0)
    assert np.allclose(g - g[0], logits - logits[0])


def test_sampler_chain_statistics_mirostat_beam_and_stops():
    cfg = S.GenerationConfig(temperature=1.0, top_k=3, seed=0)
    chain = S.SamplerChain(cfg)
    logits = np.array([2.0, 1.0, 0.5, 0.0, -1.0])
    draws = np.bincount([chain.sample(logits) for _ in range(4000)], minlength=5)
    assert draws[3:].sum() == 0 and np.allclose(draws[:3] / 4000, S.softmax(logits[:3]), atol=0.03)
    assert S.SamplerChain(S.GenerationConfig.greedy()).sample(logits) == 0
    m = S.Mirostat(tau=2.0)
    rng = np.random.default_rng(1)
    assert all(0 <= m.sample(np.random.default_rng(i).normal(size=50), rng) < 50 for i in range(20))
    det = S.StopSequenceDetector(["</s>", "STOP"])
    out = [det.push(p) for p in ["hello <", "/", "s> tail"]]
    assert out[0] == ("hello ", False) and out[1] == ("", False) and out[2] == ("", True)
    det = S.StopSequenceDetector(["END"])
    assert det.push("an E")[0] == "an " and det.push("x")[0] == "Ex"
    beam = S.BeamSearch(2, eos_token_id=0)
    lp = np.log(np.array([0.1, 0.6, 0.3]))
    beam.step([lp]); beam.step([lp, lp])
    assert beam.best().tokens == [1, 1] and len(beam.beams) == 2
    pc = S.PromptCache(2)
    pc.put([1, 2], "a"); pc.put([1, 2, 3], "b"); pc.put([9], "c")
    assert pc.get([1, 2]) is None and pc.longest_prefix([1, 2, 3, 4])[1] == "b"
    assert S.token_healing_candidates(["he", "hello", "help", "x"], "hel") == [1, 2]


def test_metrics_exposition():
    m = MetricsCollector()
    m.record_success(10, 0.5, ttft=0.05, token_times=[0.0, 0.01, 0.03]); m.record_failure()
    text = m.prometheus()
    for name in ("realizar_requests_total 2", "realizar_requests_failed 1", "realizar_tokens_generated 10", "realizar_ttft_seconds_count 1",
                 "realizar_itl_seconds_count 2", "realizar_uptime_seconds"):
        assert name in text
    assert m.snapshot()["error_rate"] == 0.5
    h = LatencyHistogram()
    for v in range(1, 101):
        h.observe(v / 1000)
    assert 0.045 <= h.percentile(50) <= 0.055 and h.percentile(99) >= 0.098
    d = DispatchMetrics(); d.record("gpu", 0.001); d.record("cpu", 0.01)
    assert d.to_dict()["gpu_dispatch_ratio"] == 0.5 and "realizar_dispatch_gpu_total 1" in d.prometheus()


# ---------------------------------------------------------------------------- HTTP -------------
@pytest.fixture(scope="module")
def client():
    from starlette.testclient import TestClient
    from realizar_b200.serving.api import AppState, create_app
    st = AppState.demo()
    with TestClient(create_app(st)) as c:
        yield c
    st.serving.stop()


def test_http_health_models_tokenize_generate(client):
    assert client.get("/health").json()["status"] == "healthy"
    assert client.get("/v1/models").json()["data"][0]["id"] == "demo"
    assert client.post("/tokenize", json={"text": "ab"}).json() == {"token_ids": [97, 98], "num_tokens": 2}
    r = client.post("/generate", json={"prompt": "a", "max_tokens": 3}).json()
    assert r["token_ids"] == [98, 99, 100] and r["text"] == "bcd" and r["num_generated"] == 3
    r = client.post("/batch/generate", json={"prompts": ["a", "x"], "max_tokens": 2}).json()
    assert [x["text"] for x in r["results"]] == ["bc", "yz"]
    assert client.get("/nope").status_code == 404 and "error" in client.get("/nope").json()
    assert client.post("/generate", json={"max_tokens": 3}).status_code == 422
    assert client.post("/generate", json={"prompt": "a", "strategy": "bogus"}).status_code == 400


def test_http_chat_completions_and_streaming(client):
    body = {"model": "demo", "messages": [{"role": "user", "content": "A"}], "max_tokens": 4, "temperature": 0}
    r = client.post("/v1/chat/completions", json=body, headers={"X-Trace-Level": "brick"}).json()
    assert r["object"] == "chat.completion" and r["choices"][0]["message"] == {"role": "assistant", "content": "BCDE"}
    assert r["choices"][0]["finish_reason"] == "length" and r["usage"] == {"prompt_tokens": 1, "completion_tokens": 4, "total_tokens": 5}
    assert "brick_trace" in r and client.get(f"/v1/audit/{r['id']}").json()["completion_tokens"] == 4
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as resp:
        events = [l[6:] for l in resp.iter_lines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "BCDE"
    assert chunks[-1]["choices"][0]["finish_reason"] == "length" and chunks[0]["object"] == "chat.completion.chunk"
    r = client.post("/v1/completions", json={"prompt": "a", "max_tokens": 2, "temperature": 0}).json()
    assert r["choices"][0]["text"] == "bc"
    m = client.get("/metrics").text
    assert "realizar_requests_total" in m and "realizar_ttft_seconds_bucket" in m
    assert client.get("/v1/metrics").json()["requests_successful"] >= 3
    assert client.get("/metrics/dispatch").json()["total_dispatches"] >= 3


def test_http_scoring_endpoints(client):
    """/v1/logprobs, /v1/perplexity and /v1/embeddings run a scoring pass on the engine thread (here the toy engine, whose
    successor token has probability 1/2)."""
    import math
    r = client.post("/v1/logprobs", json={"prompt": "abc"}).json()
    assert r["tokens"] == [97, 98, 99] and r["token_logprobs"][0] is None
    assert all(abs(x - math.log(0.5)) < 1e-9 for x in r["token_logprobs"][1:])
    p = client.post("/v1/perplexity", json={"text": "abcd"}).json()
    assert abs(p["perplexity"] - 2.0) < 1e-9 and p["num_tokens"] == 4
    assert client.post("/v1/perplexity", json={"text": "a"}).status_code == 400
    e = client.post("/v1/embeddings", json={"input": ["ab", "c"]}).json()
    assert [d["embedding"] for d in e["data"]] == [[97.5, 2.0], [99.0, 1.0]] and e["usage"]["prompt_tokens"] == 3


def test_http_stop_strings_penalties_and_grammar(client):
    """Request-level controls reach the engine: stop strings end the generation (also mid-stream, and the stop string is
    never sent), penalties and logit_bias arrive as sampling parameters, a GBNF grammar becomes per-step token masks."""
    body = {"model": "demo", "messages": [{"role": "user", "content": "A"}], "max_tokens": 12, "temperature": 0}
    r = client.post("/v1/chat/completions", json={**body, "stop": ["EF"]}).json()
    assert r["choices"][0]["message"]["content"] == "BCD" and r["choices"][0]["finish_reason"] == "stop"
    assert r["usage"]["completion_tokens"] <= 6                      # generation ended at the stop string, not at max_tokens
    with client.stream("POST", "/v1/chat/completions", json={**body, "stop": ["EF"], "stream": True}) as resp:
        events = [json.loads(l[6:]) for l in resp.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in events if "choices" in c) == "BCD"
    eng = client.app.state.rlz.serving.engine
    client.post("/v1/chat/completions", json={**body, "max_tokens": 2, "presence_penalty": 0.5, "frequency_penalty": 0.25, "repetition_penalty": 1.3,
                                              "logit_bias": {"66": -100}, "top_k": 7, "min_p": 0.05, "temperature": 0.8})
    last = [c for c in eng.calls if c[0] == "sampling"][-1]
    assert last[2] == 0.8
    got = [v for v in eng.sampling_log if v.repetition_penalty == 1.3]
    assert got and got[-1].presence_penalty == 0.5 and got[-1].frequency_penalty == 0.25 and got[-1].logit_bias == {66: -100.0} and got[-1].top_k == 7
    assert client.post("/v1/chat/completions", json={**body, "logit_bias": {"x": 1}}).status_code == 400
    # grammar: only the letters x / y may follow, so the toy engine (successor of its input) is overruled by the mask
    r = client.post("/v1/chat/completions", json={**body, "max_tokens": 4, "grammar": 'root ::= [xy]+'}).json()
    assert set(r["choices"][0]["message"]["content"]) <= set("xy") and len(r["choices"][0]["message"]["content"]) == 4
    assert any(c[0] == "mask" for c in eng.calls)
    assert client.post("/v1/chat/completions", json={**body, "grammar": "root ::= ("}).status_code == 400
    r = client.post("/v1/completions", json={"prompt": "a", "max_tokens": 8, "temperature": 0, "stop": ["de"]}).json()
    assert r["choices"][0]["text"] == "bc" and r["choices"][0]["finish_reason"] == "stop"


def test_trace_context_is_propagated_and_requests_are_recorded():
    from fastapi.testclient import TestClient
    from realizar_b200.serving.api import AppState, create_app
    state = AppState.demo()
    try:
        with TestClient(create_app(state)) as c:
            tid = "4bf92f3577b34da6a3ce929d0e0e4736"
            r = c.get("/health", headers={"traceparent": f"00-{tid}-00f067aa0ba902b7-01"})
            assert r.status_code == 200 and r.headers["traceparent"].split("-")[1] == tid      # same trace, new span id
            assert r.headers["traceparent"].split("-")[2] != "00f067aa0ba902b7"
            r2 = c.get("/health")                                                             # no header: a new trace is started
            assert len(r2.headers["traceparent"].split("-")[1]) == 32 and r2.headers["traceparent"].split("-")[1] != tid
            spans = c.get("/v1/traces").json()["spans"]
            assert spans[0]["traceId"] == tid and spans[0]["parentSpanId"] == "00f067aa0ba902b7" and spans[0]["name"] == "GET /health"
            lat = c.get("/v1/metrics").json()["http_latency_ms"]
            assert lat["/health"]["count"] == 2
            sched = c.get("/v1/metrics").json()["scheduler"]
            assert "requests_done" in sched
    finally:
        state.serving.stop()


def test_recovery_after_a_failed_step_and_refusal_when_the_context_is_lost():
    """The engine raises in the middle of serving: requests in flight fail, /health turns unhealthy; POST /v1/gpu/reset resets the
    engine in place and the server answers again; when the reset probe itself fails (device context lost) the latch stays."""
    from fastapi.testclient import TestClient
    from realizar_b200.runtime.scheduler import FakeEngine, ServingEngine
    from realizar_b200.serving.api import AppState, create_app
    from realizar_b200.serving.chat_template import RawTemplate
    from realizar_b200.serving.tokenizer import ByteTokenizer
    eng = FakeEngine(vocab=256, fail_after=3)
    serving = ServingEngine(eng).start()
    state = AppState(serving, ByteTokenizer(256), RawTemplate(), "demo", None, compute_mode="cpu")
    try:
        with TestClient(create_app(state)) as c:
            r = c.post("/generate", json={"prompt": "abc", "max_tokens": 20})
            assert r.status_code == 500
            for _ in range(100):
                if serving.health != "ok":
                    break
                time.sleep(0.01)
            assert c.get("/health").status_code == 503
            eng.fail_after = None
            assert c.post("/v1/gpu/reset").json() == {"status": "ok", "health": "ok"}
            assert c.get("/health").status_code == 200
            ok = c.post("/generate", json={"prompt": "abc", "max_tokens": 5})
            assert ok.status_code == 200 and ok.json()["num_generated"] == 5
            # second failure, and this time the device does not answer the probe
            eng.fail_after, eng.steps = 1, 0
            assert c.post("/generate", json={"prompt": "abc", "max_tokens": 20}).status_code == 500
            for _ in range(100):
                if serving.health != "ok" and not serving._thread.is_alive():
                    break
                time.sleep(0.01)
            eng.context_lost = True
            r = c.post("/v1/gpu/reset")
            assert r.status_code == 503 and "context lost" in r.json()["detail"]
            assert c.get("/health").status_code == 503
    finally:
        serving.stop()


def test_token_fanout_coalesces_wakeups_and_keeps_order():
    """Many posts from another thread between two runs of the event loop arrive through ONE scheduled drain, in order."""
    import asyncio
    from realizar_b200.serving.api import TokenFanout

    async def main():
        loop = asyncio.get_running_loop()
        fan = TokenFanout(loop)
        q1, q2 = asyncio.Queue(), asyncio.Queue()
        calls = []
        orig = loop.call_soon_threadsafe
        loop.call_soon_threadsafe = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]

        def producer():
            for i in range(100):
                fan.post(q1 if i % 2 == 0 else q2, ("tok", i))
            fan.post(q1, ("end", None))
        t = threading.Thread(target=producer)
        t.start()
        t.join()                                             # the loop has not run in between: everything is pending
        got1 = [await q1.get() for _ in range(51)]
        got2 = [await q2.get() for _ in range(50)]
        assert [v for _, v in got1[:-1]] == list(range(0, 100, 2)) and got1[-1] == ("end", None)
        assert [v for _, v in got2] == list(range(1, 100, 2))
        assert len(calls) == 1                               # one wake-up for 101 posts
        fan.post(q2, ("tok", 7))                             # and the next burst schedules its own
        assert await q2.get() == ("tok", 7) and len(calls) == 2
    asyncio.run(main())
