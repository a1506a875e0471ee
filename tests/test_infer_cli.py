"""High-level inference, CLI commands, registry/cache/warm-up/URIs, resilience, stats and bench utilities."""
import io
import json
import os

import numpy as np
import pytest

from realizar_b200 import cli
from realizar_b200.infer import InferenceConfig, LLM, run_inference, validate_model_path
from realizar_b200.models.config import named_config
from realizar_b200.models.cpu_model import CpuModel
from realizar_b200.models.weights import synthetic_weights, weights_to_gguf
from realizar_b200.runtime import registry as R
from realizar_b200.runtime import resilience as Z
from realizar_b200.serving.tokenizer import bytes_to_unicode
from realizar_b200.utils import benchlib, stats, viz
from realizar_b200.utils.trace import BrickProfiler, InferenceTracer, TensorStats, compare_traces, first_divergence


@pytest.fixture(scope="module")
def gguf_path(tmp_path_factory):
    w = synthetic_weights(named_config("tiny-llama"), seed=0, std=0.05)
    b2u = bytes_to_unicode()
    vocab = [b2u[i] for i in range(256)] + [f"<t{i}>" for i in range(256)]
    p = tmp_path_factory.mktemp("m") / "tiny.gguf"
    p.write_bytes(weights_to_gguf(w, vocabulary=vocab))
    return str(p), w


def test_run_inference_cpu_matches_engine(gguf_path):
    path, w = gguf_path
    r = run_inference(InferenceConfig(path, prompt="hello", max_tokens=6, use_gpu=False, trace=True))
    assert r.format == "gguf" and not r.used_gpu and r.generated_token_count == 6 and r.input_token_count == 5
    assert r.tok_per_sec > 0 and r.load_ms > 0
    ref, _, _ = CpuModel(w, 64).generate_greedy(r.tokens[:5], 6, None)
    assert r.tokens[5:] == list(ref)
    names = [e["details"]["name"] for e in r.trace_events]
    assert names[:2] == ["LOAD", "LOAD"] and "TOKENIZE" in names and "DECODE" in names
    assert {e["type"] for e in r.trace_events} == {"TaskStateEntered", "TaskStateExited"}


def test_run_inference_errors(tmp_path, gguf_path):
    with pytest.raises(FileNotFoundError):
        validate_model_path(str(tmp_path / "missing.gguf"))
    bad = tmp_path / "m.txt"
    bad.write_text("x")
    with pytest.raises(ValueError):
        validate_model_path(str(bad))
    with pytest.raises(ValueError):
        run_inference(InferenceConfig(gguf_path[0], use_gpu=False))


def test_llm_sampling_and_token_input(gguf_path):
    llm = LLM(gguf_path[0], use_gpu=False, max_seq_len=64)
    out = llm.generate_tokens([1, 2, 3], max_tokens=5, temperature=0.8, top_k=10)
    assert len(out) <= 5 and all(0 <= t < llm.cfg.vocab_size for t in out)
    r = run_inference(InferenceConfig(gguf_path[0], input_tokens=[1, 2, 3], max_tokens=3, use_gpu=False))
    assert r.input_token_count == 3


def test_cli_run_info_convert(gguf_path, tmp_path, capsys):
    path, _ = gguf_path
    assert cli.main(["run", path, "hi", "--no-gpu", "-n", "4", "--raw", "--format", "json", "--temperature", "0"]) == 0
    d = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert d["tokens_generated"] == 4 and d["format"] == "gguf" and d["used_gpu"] is False
    assert cli.main(["info", path]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["architecture"] == "llama" and info["layers"] == 2
    dst = str(tmp_path / "o.apr")
    assert cli.main(["convert", path, dst, "--to", "apr"]) == 0
    capsys.readouterr()
    assert cli.main(["run", dst, "hi", "--no-gpu", "-n", "4", "--raw", "--format", "json", "--temperature", "0"]) == 0
    d2 = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert d2["format"] == "apr" and d2["text"] == d["text"]
    assert cli.main(["run", str(tmp_path / "nope.gguf"), "x"]) == 1


def test_cli_chat_loop(gguf_path, tmp_path):
    path, _ = gguf_path
    a = cli.build_parser().parse_args(["chat", path, "--no-gpu", "-n", "3", "--temperature", "0", "--history", str(tmp_path / "h.json")])
    out = io.StringIO()
    assert cli.cmd_chat(a, stdin=io.StringIO("hello\n/history\n/clear\n\n/exit\n"), stdout=out) == 0
    assert ">>> " in out.getvalue()
    assert json.loads((tmp_path / "h.json").read_text()) == []
    h = []
    assert cli.process_chat_input("/quit", h) == "exit" and cli.process_chat_input("  ", h) == "handled" and cli.process_chat_input("hi", h) is None


def test_cli_bench_compare_list_viz(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("REALIZAR_HOME", str(tmp_path))
    (tmp_path / "models" / "org").mkdir(parents=True)
    (tmp_path / "models" / "org" / "m.gguf").write_bytes(b"GGUF" + b"\0" * 100)
    assert cli.main(["list", "--format", "json"]) == 0
    assert json.loads(capsys.readouterr().out)[0]["name"] == "org/m.gguf"
    assert R.resolve_uri("pacha://org/m").name == "m.gguf"
    assert cli.main(["pull", "x"]) == 2
    f1, f2 = str(tmp_path / "a.json"), str(tmp_path / "b.json")
    rng = np.random.default_rng(0)
    benchlib.save_results(f1, [benchlib.BenchResult("lat", "ms", list(rng.normal(10, 0.2, 30)))])
    benchlib.save_results(f2, [benchlib.BenchResult("lat", "ms", list(rng.normal(13, 0.2, 30)))])
    assert cli.main(["bench-compare", f1, f2]) == 0
    assert "regressed" in capsys.readouterr().out
    assert cli.main(["bench-regression", f1, f2]) == 1
    assert cli.main(["bench-regression", f2, f1]) == 0
    assert cli.main(["viz", f1]) == 0 and "p99" in capsys.readouterr().out
    assert cli.main(["bench", "--list"]) == 0
    assert cli.main(["bench", "cache", "-o", str(tmp_path / "c.json")]) == 0
    assert cli.main(["bench", "cpu_generate", "--model", "tiny-llama", "-o", str(tmp_path / "g.json")]) == 0       # 128 + 128 tokens on the CPU engine
    names = [r["name"] for r in json.loads((tmp_path / "g.json").read_text())["results"]] if (tmp_path / "g.json").exists() else []
    assert any("decode_tok_per_s" in n for n in names) and any("prompt_tok_per_s" in n for n in names), names
    assert "paged_kv_open_reserve_close_64x512" in benchlib.load_results(str(tmp_path / "c.json"))


def test_serving_stress_tests_on_fake_engine():
    from realizar_b200.runtime.scheduler import FakeEngine, ServingEngine
    s = ServingEngine(FakeEngine(vocab=1000)).start()
    try:
        c = benchlib.convoy_test(s, vocab=900)
        assert c["ok"] and c["completed"] == c["total"] and not c["hol_blocking"]
        sat = benchlib.saturation_test(s, concurrency=8, requests=24, vocab=900)
        assert sat["completed"] + sat["rejected"] == 24 and sat["tok_per_s"] > 0
    finally:
        s.stop()


def test_cpu_slot_engine_serves(gguf_path):
    from realizar_b200.runtime.cpu_engine import CpuEngineConfig, CpuSlotEngine
    from realizar_b200.runtime.scheduler import ServingEngine
    _, w = gguf_path
    s = ServingEngine(CpuSlotEngine(w, CpuEngineConfig(2, 64))).start()
    try:
        r = s.generate([1, 2, 3, 4], timeout=30, max_tokens=5, temperature=0.0)
        ref, _, _ = CpuModel(w, 64).generate_greedy([1, 2, 3, 4], 5, None)
        assert r.output == list(ref)
    finally:
        s.stop()


# -- registry / cache / warm-up / uri --------------------------------------------------------------
def test_registry_and_cache():
    reg = R.ModelRegistry()
    reg.register("a", object(), "tokA")
    reg.register("b", object())
    assert reg.default_id == "a" and reg.get()[1] == "tokA" and len(reg) == 2 and reg.contains("b")
    with pytest.raises(R.RegistryError):
        reg.register("a", object())
    new = object()
    reg.replace("a", new)
    assert reg.get("a")[0] is new
    reg.unregister("a")
    assert reg.default_id == "b"
    with pytest.raises(R.RegistryError):
        reg.get("zzz")
    ev = []
    c = R.ModelCache(2, on_evict=lambda k, v: ev.append(k))
    loads = []
    for k in ("x", "y", "x", "z", "y"):
        c.get_or_load(k, lambda k=k: loads.append(k) or k.upper())
    assert loads == ["x", "y", "z", "y"] and ev == ["y", "x"] and c.metrics.hits == 1 and c.metrics.evictions == 2
    with pytest.raises(RuntimeError):
        c.get_or_load("boom", lambda: (_ for _ in ()).throw(RuntimeError("load failed")))
    assert c.get_or_load("boom", lambda: 1) == 1


def test_warmup_and_uri(tmp_path):
    calls = []
    h = R.ModelHealth()
    res = R.ModelWarmer(R.WarmupConfig(iterations=3)).warm(lambda p, n: calls.append((len(p), n)), 100, h)
    assert res.success and res.iterations_completed == 3 and calls == [(8, 4)] * 3 and h.is_ready
    bad = R.ModelWarmer().warm(lambda p, n: 1 / 0, 100, h)
    assert not bad.success and "ZeroDivision" in bad.error and h.state == "degraded"
    u = R.ModelUri.parse("pacha://model/llama3:1.0")
    assert (u.scheme, u.name, u.version) == ("pacha", "llama3", "1.0") and str(u) == "pacha://llama3:1.0"
    for bad_uri in ("", "ftp://x", "pacha://", "pacha://a:", "pacha://../etc"):
        with pytest.raises(ValueError):
            R.ModelUri.parse(bad_uri)
    with pytest.raises(FileNotFoundError):
        R.resolve_uri("pacha://nothing", tmp_path)


# -- resilience ----------------------------------------------------------------------------------------
def test_retry_and_circuit_breaker():
    sleeps, n = [], [0]

    def flaky():
        n[0] += 1
        if n[0] < 3:
            raise TimeoutError("t")
        return "ok"
    assert Z.RetryPolicy(Z.RetryConfig(3, 0.1, jitter=0.0)).run(flaky, sleeps.append) == "ok" and sleeps == [0.1, 0.2]
    with pytest.raises(ValueError):
        Z.RetryPolicy().run(lambda: (_ for _ in ()).throw(ValueError("permanent")), sleeps.append)
    assert Z.categorize(MemoryError()) == Z.ErrorCategory.OVERLOAD
    now = [0.0]
    cb = Z.CircuitBreaker(2, 1, 10.0, clock=lambda: now[0])
    for _ in range(2):
        with pytest.raises(RuntimeError):
            cb.call(lambda: (_ for _ in ()).throw(RuntimeError("x")))
    assert cb.state == Z.CircuitState.OPEN
    with pytest.raises(Z.CircuitOpen):
        cb.call(lambda: 1)
    now[0] = 11.0
    assert cb.call(lambda: 7) == 7 and cb.state == Z.CircuitState.CLOSED


def test_bulkhead_limits_and_misc():
    b = Z.Bulkhead({"inference": 1, "batch": 1})
    assert b.try_acquire("inference") and not b.try_acquire("inference") and b.try_acquire("batch")
    with pytest.raises(Z.BulkheadFull):
        b.run("inference", lambda: 1)
    b.release("inference")
    assert b.run("inference", lambda: 5) == 5 and b.available("inference") == 1
    now = [0.0]
    tm = Z.TimeoutManager(lambda: now[0])
    tm.register("a", 1.0); tm.register("b", 5.0)
    now[0] = 2.0
    assert tm.expired() == ["a"] and tm.expired() == []
    rl = Z.TokenRateLimiter(10.0, 5.0, lambda: now[0])
    assert all(rl.try_acquire() for _ in range(5)) and not rl.try_acquire()
    now[0] = 2.5
    assert rl.try_acquire(4)
    rt = Z.ResourceTracker(100, 2)
    a1 = rt.allocate(60)
    assert a1 and rt.allocate(60) is None and rt.allocate(30) and rt.allocate(1) is None
    rt.release(a1)
    assert rt.usage() == (0.3, 0.5)
    q = Z.PriorityRequestQueue()
    q.push("lo", 0); q.push("hi", 5); q.push("hi2", 5)
    assert [q.pop(), q.pop(), q.pop(), q.pop()] == ["hi", "hi2", "lo", None]
    sc = Z.ShutdownCoordinator()
    ran = []
    sc.register_handler(lambda: ran.append(1))
    assert sc.request_started()
    sc.request_completed()
    assert sc.initiate(0.1) and ran == [1] and not sc.request_started()
    hc = Z.HealthChecker()
    hc.register("ok", lambda: True); hc.register("bad", lambda: 1 / 0)
    assert hc.check_all() == {"ok": True, "bad": False} and not hc.healthy


# -- stats / viz / bench ----------------------------------------------------------------------------------
def test_stats_against_scipy():
    import scipy.stats as ss
    rng = np.random.default_rng(1)
    a, b = rng.normal(10, 1, 40), rng.normal(10.8, 1.5, 35)
    w = stats.welch_t_test(a, b)
    assert abs(w.p_value - ss.ttest_ind(a, b, equal_var=False).pvalue) < 1e-9
    m = stats.mann_whitney_u(a, b)
    assert abs(m.p_value - ss.mannwhitneyu(a, b).pvalue) < 1e-6
    assert stats.analyze_with_auto_select(a, b).method == "welch"
    assert stats.analyze_with_auto_select(rng.lognormal(0, 2, 40), b).method == "mann-whitney"
    lo, hi = stats.bootstrap_ci(a)
    assert lo < a.mean() < hi
    s = stats.summarize(a)
    assert s.n == 40 and s.min <= s.p50 <= s.p95 <= s.p99 <= s.max


def test_dynamic_sampler_thermal_itl_viz():
    vals = iter([10, 30, 5, 20] + [10.0] * 100)
    ds = benchlib.DynamicSampler(min_samples=4, max_samples=50, cv_threshold=0.05, window=5)
    out = ds.run(lambda: next(vals))
    assert 8 <= len(out) < 50 and ds.current_cv() <= 0.05
    tg = benchlib.ThermalGuard(80, 70, 1.0, 10)
    temps = iter([85, 78, 69])
    slept = []
    assert tg.needs_cooldown(85) and tg.cooldown(lambda: next(temps), slept.append) == 2.0
    tg.record(60); tg.record(75)
    assert not tg.is_valid_run()
    itl = benchlib.ItlMetrics.from_timestamps([0.0, 0.01, 0.02, 0.05])
    assert abs(itl.median_ms - 10) < 1e-6 and itl.p99_ms > 25
    assert viz.sparkline([1, 2, 3]) == "▁▅█" and len(viz.sparkline(range(100), 10)) == 10
    assert "█" in viz.histogram([1, 1, 2, 5]) and "b" in viz.bar_table({"a": 1.0, "b": 2.0})


def test_tracing_tools():
    t = InferenceTracer()
    t.enter("EMBED", tokens=3); t.tensor("EMBED", "x", np.array([1.0, np.nan, np.inf])); t.exit("EMBED", dim=8)
    ev = json.loads(t.to_json())["events"]
    assert [e["type"] for e in ev] == ["TaskStateEntered", "TensorStats", "TaskStateExited"] and ev[1]["details"]["nan_count"] == 1
    assert "EMBED" in t.summary()
    off = InferenceTracer(False); off.enter("X"); off.exit("X")
    assert off.events == []
    ts = TensorStats.of(np.arange(10.0))
    assert ts.healthy and ts.mean == 4.5 and ts.size == 10
    a = {"l0": np.ones(8), "l1": np.arange(8.0)}
    b = {"l0": np.ones(8), "l1": -np.arange(8.0)}
    d = compare_traces(a, b)
    assert d[0].ok and not d[1].ok and first_divergence(d).name == "l1"
    bp = BrickProfiler(cuda=False)
    with bp.brick("a"):
        sum(range(1000))
    with bp.brick("a"):
        pass
    assert bp.summary()["a"]["count"] == 2 and bp.bottleneck() == "a"


def test_monitor_renders():
    from realizar_b200.utils.tui import run_monitor
    out = []
    rc = run_monitor("http://x", once=True, fetch=lambda u: {"tokens_per_sec": 123.0, "latency_p50_ms": 5, "total_requests": 3}, out=out.append)
    assert rc == 0 and "123.0 tok/s" in out[0] and "total 3" in out[0]
    assert run_monitor("http://x", once=True, fetch=lambda u: 1 / 0, out=out.append) == 1


def test_targets_and_http_client_and_bricks():
    from realizar_b200.utils.bricks import TokenBudget, TransformerLayerBrick
    from realizar_b200.utils.http_client import ModelHttpClient
    from realizar_b200.utils.target import BuildManifest, DeployTarget, DockerConfig, TargetCapabilities
    assert DeployTarget.detect({"AWS_LAMBDA_FUNCTION_NAME": "f"}) == DeployTarget.LAMBDA
    assert DeployTarget.detect({"KUBERNETES_SERVICE_HOST": "h"}) == DeployTarget.KUBERNETES
    assert not TargetCapabilities.of(DeployTarget.LAMBDA).supports("gpu") and TargetCapabilities.of(DeployTarget.NATIVE).supports("multi_gpu")
    df = DockerConfig(model_path="m/phi2.gguf").generate_dockerfile()
    assert df.startswith("FROM nvidia/cuda") and "/models/phi2.gguf" in df and "EXPOSE 8080" in df
    assert "sm_100a" in BuildManifest.default("0.1").to_json()
    sent = []

    def transport(url, body, timeout):
        sent.append((url, body))
        return {"choices": [{"text": "hi", "message": {"content": "yo"}}], "usage": {"completion_tokens": 7}, "response": "r", "eval_count": 3}
    c = ModelHttpClient("http://h:1/", transport=transport)
    assert c.openai_completion("m", "p").tokens_generated == 7 and c.openai_chat("m", [{"role": "user", "content": "x"}]).text == "yo"
    assert c.ollama_generate("m", "p").tokens_generated == 3 and sent[2][0] == "http://h:1/api/generate"
    assert TokenBudget.from_throughput(1000).us_per_token == 1000 and abs(TokenBudget.from_bytes(6.5e6, 6500).us_per_token - 1.0) < 1e-9
    lb = TransformerLayerBrick.from_model_shape(2560, 2560, 2560, 10240, 4.5, 512, 6500)
    lb.record({"QkvProjection": 1.0, "GateUpProjection": 500.0, "AttentionScore": 2.0})
    bn = lb.bottleneck()
    assert bn.brick == "GateUpProjection" and bn.gap > 1 and lb.total_budget_us() > 0
    assert any(not v.passed for v in lb.verify())


def test_load_generator_inprocess(capsys):
    from realizar_b200.serving.api import AppState, create_app
    from realizar_b200.utils.loadgen import LoadConfig, run_load
    st = AppState.demo()
    try:
        r = run_load(LoadConfig(requests=12, rate_per_s=500, max_concurrency=4, prompt_tokens=6, max_tokens=5), app=create_app(st))
    finally:
        st.serving.stop()
    # (the demo engine produces a request's tokens faster than the loop delivers them, so they may arrive as one event each:
    # the count of generated tokens comes from the stream's usage record, inter-token gaps exist only between separate events)
    assert r["completed"] == 12 and r["errors"] == 0 and r["tokens"] == 12 * 5 and r["events"] >= 12 and r["ttft_ms"]["p50"] is not None
    assert cli.main(["bench-serving", "--requests", "6", "--rate", "0", "--concurrency", "3", "--max-tokens", "4", "--prompt-tokens", "4"]) == 0
    assert json.loads(capsys.readouterr().out)["completed"] == 6
