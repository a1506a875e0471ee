"""Command line: ``run``, ``chat``, ``serve``, ``list``, ``pull``/``push`` (offline: explain),
``bench``, ``bench-convoy``, ``bench-saturation``, ``bench-compare``, ``bench-regression``, ``viz``,
``convert``, ``monitor`` and ``info``.  ``python -m realizar_b200 <command>``.
Reference parity: ``Commands`` (src/cli/handlers.rs:25-290), ``run_gguf_inference`` and friends
(src/cli/inference.rs), ``serve_model`` (src/cli/mod_server_commands.rs:361-476)."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import List, Optional


def format_size(n: int) -> str:
    for unit, s in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if n >= s:
            return f"{n / s:.1f} {unit}"
    return f"{n} B"


def _add_gen_args(p):
    p.add_argument("--max-tokens", "-n", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--system", default=None)
    p.add_argument("--gpu", dest="gpu", action="store_true", default=None)
    p.add_argument("--no-gpu", dest="gpu", action="store_false")
    p.add_argument("--max-seq-len", type=int, default=4096)
    p.add_argument("--kv-dtype", choices=["bf16", "q8"], default="bf16", help="KV cache rows on the GPU engine")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="realizar-b200", description="B200-native LLM inference: run, chat, serve, benchmark, convert")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="generate from a prompt")
    r.add_argument("model"); r.add_argument("prompt", nargs="?"); _add_gen_args(r)
    r.add_argument("--raw", action="store_true", help="no chat template"); r.add_argument("--format", choices=["text", "json"], default="text")
    r.add_argument("--trace", nargs="?", const="-", default=None, help="emit step trace (optionally to a file)"); r.add_argument("--verbose", "-v", action="store_true")
    c = sub.add_parser("chat", help="interactive chat"); c.add_argument("model"); _add_gen_args(c); c.add_argument("--history", default=None)
    s = sub.add_parser("serve", help="HTTP server with the OpenAI-compatible API")
    s.add_argument("--model", default=None); s.add_argument("--host", default="127.0.0.1"); s.add_argument("--port", type=int, default=8080)
    s.add_argument("--demo", action="store_true"); s.add_argument("--max-batch", type=int, default=4); s.add_argument("--max-seq-len", type=int, default=4096)
    s.add_argument("--gpu", dest="gpu", action="store_true", default=None); s.add_argument("--no-gpu", dest="gpu", action="store_false")
    s.add_argument("--kv-dtype", choices=["bf16", "q8"], default="bf16"); s.add_argument("--no-warmup", action="store_true"); s.add_argument("--classical", default=None, help="classical-ML .apr model behind /v1/predict")
    s.add_argument("--tp-comm", choices=["fused", "nccl"], default="fused", help="tensor parallel (under torch.distributed.run): in-kernel collectives or NCCL")
    s.add_argument("--draft-layers", type=int, default=0, help="self-speculative decoding for lone greedy streams: layers in the draft (0 = off)")
    s.add_argument("--prefill-chunk", type=int, default=256, help="prompt tokens run between two decode steps")
    l = sub.add_parser("list", help="models in the local store"); l.add_argument("--format", choices=["table", "json"], default="table")
    for name in ("pull", "push"):
        q = sub.add_parser(name, help=f"{name} a model ({'needs a network' })"); q.add_argument("model")
    b = sub.add_parser("bench", help="kernel / engine benchmarks")
    b.add_argument("suite", nargs="?", default=None, help="quantize | cpu_decode | cpu_generate | tokenizer | cache | decode (GPU) | gemv | gemm | attn")
    b.add_argument("--list", action="store_true"); b.add_argument("--output", "-o", default=None); b.add_argument("--model", default="tiny-llama")
    for name in ("bench-convoy", "bench-saturation"):
        q = sub.add_parser(name); q.add_argument("--model", default=None); q.add_argument("--output", "-o", default=None)
        q.add_argument("--concurrency", type=int, default=16); q.add_argument("--requests", type=int, default=64)
    bs = sub.add_parser("bench-serving", help="open-loop load against the OpenAI API (Poisson arrivals, SSE streaming)")
    bs.add_argument("--url", default=None, help="running server; default: load the model in-process"); bs.add_argument("--model", default=None)
    bs.add_argument("--requests", type=int, default=200); bs.add_argument("--rate", type=float, default=20.0); bs.add_argument("--concurrency", type=int, default=256)
    bs.add_argument("--prompt-tokens", type=int, default=64); bs.add_argument("--max-tokens", type=int, default=32); bs.add_argument("--max-batch", type=int, default=64)
    bs.add_argument("--prompt-tokens-max", type=int, default=0, help="> --prompt-tokens: prompt lengths uniform in that range")
    bs.add_argument("--prompt-chars", action="store_true", help="count prompt length in characters (byte-level tokenizers: tokens)")
    bs.add_argument("--temperature", type=float, default=0.0); bs.add_argument("--top-p", type=float, default=1.0)
    bs.add_argument("--http", action="store_true", help="serve the in-process model on a local port and drive it over real HTTP")
    bs.add_argument("--port", type=int, default=18080); bs.add_argument("--max-seq-len", type=int, default=4096)
    bs.add_argument("--tp-comm", choices=["fused", "nccl"], default="fused"); bs.add_argument("--prefill-chunk", type=int, default=256)
    bs.add_argument("--output", "-o", default=None)
    bc = sub.add_parser("bench-compare"); bc.add_argument("file1"); bc.add_argument("file2"); bc.add_argument("--threshold", type=float, default=5.0)
    br = sub.add_parser("bench-regression"); br.add_argument("baseline"); br.add_argument("current"); br.add_argument("--strict", action="store_true")
    v = sub.add_parser("viz"); v.add_argument("file", nargs="?"); v.add_argument("--samples", type=int, default=100)
    cv = sub.add_parser("convert"); cv.add_argument("src"); cv.add_argument("dst"); cv.add_argument("--to", choices=["apr", "gguf"], default="apr")
    cv.add_argument("--qtype", default=None); cv.add_argument("--compression", choices=["lz4", "zstd"], default=None)
    m = sub.add_parser("monitor"); m.add_argument("--url", default="http://127.0.0.1:8080"); m.add_argument("--interval", type=float, default=1.0); m.add_argument("--once", action="store_true")
    i = sub.add_parser("info"); i.add_argument("model", nargs="?")
    return ap


# -- commands -------------------------------------------------------------------------------------
def cmd_run(a) -> int:
    from .infer import InferenceConfig, run_inference
    from .runtime.registry import resolve_uri
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    cfg = InferenceConfig(str(resolve_uri(a.model)), prompt=prompt, max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                          use_gpu=a.gpu, chat=not a.raw, system_prompt=a.system, trace=a.trace is not None,
                          trace_output=None if a.trace in (None, "-") else a.trace, max_seq_len=a.max_seq_len, verbose=a.verbose, kv_dtype=a.kv_dtype)
    r = run_inference(cfg)
    if a.format == "json":
        print(json.dumps({"text": r.text, "tokens_generated": r.generated_token_count, "input_tokens": r.input_token_count, "inference_ms": r.inference_ms,
                          "tok_per_sec": r.tok_per_sec, "load_ms": r.load_ms, "format": r.format, "used_gpu": r.used_gpu}))
    else:
        print(r.text)
        if a.verbose:
            print(f"[{r.format} {'gpu' if r.used_gpu else 'cpu'}] load {r.load_ms:.0f} ms, {r.generated_token_count} tokens in {r.inference_ms:.0f} ms "
                  f"({r.tok_per_sec:.1f} tok/s)", file=sys.stderr)
    if a.trace == "-":
        print(json.dumps({"events": r.trace_events}), file=sys.stderr)
    return 0


def process_chat_input(line: str, history: list) -> Optional[str]:
    """Slash commands of the chat loop.  Returns "exit", "handled" or None (a normal message)."""
    s = line.strip()
    if s in ("/exit", "/quit", "exit", "quit"):
        return "exit"
    if s == "/clear":
        history.clear()
        return "handled"
    if s == "/history":
        for m in history:
            print(f"{m.role}: {m.content}")
        return "handled"
    return "handled" if not s else None


def cmd_chat(a, stdin=None, stdout=None) -> int:
    from .infer import LLM
    from .runtime.registry import resolve_uri
    from .serving.chat_template import ChatMessage
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    llm = LLM(str(resolve_uri(a.model)), a.gpu, a.max_seq_len, max_batch=1, kv_dtype=a.kv_dtype)
    history: list = [ChatMessage.system(a.system)] if a.system else []
    print(f"model {llm.path.name} ({llm.format}, {'gpu' if llm.used_gpu else 'cpu'}); /exit to quit, /clear to reset", file=stdout)
    while True:
        print(">>> ", end="", file=stdout, flush=True)
        line = stdin.readline()
        if not line:
            break
        act = process_chat_input(line, history)
        if act == "exit":
            break
        if act == "handled":
            continue
        history.append(ChatMessage.user(line.strip()))
        ids = llm.tokenizer.encode(llm.template.format_conversation(history))[-(llm.max_seq_len - a.max_tokens - 1):]
        pieces: List[int] = []

        def on_tok(t, pieces=pieces):
            if t == llm.cfg.eos_token_id:
                return
            before = llm.tokenizer.decode(pieces)
            pieces.append(t)
            print(llm.tokenizer.decode(pieces)[len(before):], end="", file=stdout, flush=True)
        llm.generate_tokens(ids, a.max_tokens, a.temperature, a.top_k, a.top_p, on_token=on_tok)
        print(file=stdout)
        history.append(ChatMessage.assistant(llm.tokenizer.decode(pieces)))
    if a.history:
        Path(a.history).write_text(json.dumps([{"role": m.role, "content": m.content} for m in history], indent=1))
    return 0


def build_app_state(model: Optional[str], use_gpu: Optional[bool], max_batch: int, max_seq_len: int, warmup: bool = True, kv_dtype: str = "bf16",
                    tp_comm: str = "fused", draft_layers: int = 0, prefill_chunk: int = 256):
    """Load a model and wire engine -> continuous-batching loop -> API state.  Under ``torch.distributed.run`` with several
    processes the engine is tensor parallel: rank 0 returns the state, the other ranks serve rank 0's engine calls until it
    shuts down and then exit.  ``draft_layers`` > 0 turns on self-speculative decoding for lone greedy streams (that many
    evenly spaced layers form the draft); ``prefill_chunk`` bounds the prompt tokens run between two decode steps."""
    import torch
    from .formats.detect import load_model
    from .infer import build_template, build_tokenizer
    from .runtime.registry import ModelHealth, ModelWarmer, WarmupConfig, resolve_uri
    from .runtime.scheduler import SchedulerConfig, ServingEngine
    from .serving.api import AppState
    if model is None:
        return AppState.demo()
    if model.startswith("synthetic:"):
        # "synthetic:<named shape>[:<scheme>]": random-initialised weights of a named architecture (benchmarks without checkpoints)
        from .models.config import named_config
        from .models.weights import synthetic_weights
        from .serving.tokenizer import ByteTokenizer
        parts = model.split(":")
        cfg = named_config(parts[1])
        gpu = torch.cuda.is_available() if use_gpu is None else use_gpu
        w = synthetic_weights(cfg, scheme=parts[2] if len(parts) > 2 else "Q4_K_M", seed=0, device="cuda" if gpu else "cpu")
        path = Path(parts[1])
        tok_override = ByteTokenizer(cfg.vocab_size, None)
    else:
        path = resolve_uri(model)
        w = load_model(path)
        tok_override = None
    gpu = torch.cuda.is_available() if use_gpu is None else use_gpu
    msl = min(max_seq_len, w.config.context_length)
    tp_world = int(os.environ.get("WORLD_SIZE", "1")) if gpu else 1
    if gpu and tp_world > 1:
        # one process per GPU under torch.distributed.run: rank 0 serves, the other ranks follow its engine calls and never return
        from .parallel.tp_serving import TpLeaderEngine, follower_loop, init_tp, leave_group
        from .runtime.engine import DecodeEngine, EngineConfig
        rank, world, dev, comm, group = init_tp(tp_comm)
        inner = DecodeEngine(w, EngineConfig(max_batch=max_batch, max_seq_len=msl, kv_dtype=kv_dtype), device=dev, comm=comm, tp_rank=rank, tp_size=world)
        if rank != 0:
            calls = follower_loop(inner, group)
            leave_group(inner, comm)
            print(f"rank {rank}: served {calls} engine calls", file=sys.stderr)
            raise SystemExit(0)
        eng = TpLeaderEngine(inner, group, comm)
    elif gpu:
        from .runtime.engine import DecodeEngine, EngineConfig
        eng = DecodeEngine(w, EngineConfig(max_batch=max_batch, max_seq_len=msl, kv_dtype=kv_dtype))
    else:
        from .runtime.cpu_engine import CpuEngineConfig, CpuSlotEngine
        eng = CpuSlotEngine(w, CpuEngineConfig(max_batch=min(max_batch, 2), max_seq_len=msl))
    layers = None
    if draft_layers and gpu:
        n_layers = w.config.num_layers
        layers = tuple(sorted(set(range(0, n_layers, max(1, n_layers // max(1, draft_layers)))) | {n_layers - 1}))
    serving = ServingEngine(eng, SchedulerConfig(max_batch=eng.cfg.max_batch, max_seq_len=eng.cfg.max_seq_len, prefill_chunk=prefill_chunk,
                                                 token_budget=max(prefill_chunk, eng.cfg.max_batch) + eng.cfg.max_batch),
                            draft_layers=layers).start()
    st = AppState(serving, tok_override or build_tokenizer(w), build_template(w, path.stem), path.stem, None if tok_override else w.config.eos_token_id,
                  compute_mode="gpu" if gpu else "cpu",
                  context_length=eng.cfg.max_seq_len)
    if gpu:
        from .runtime.scorer import scorer_for
        st.scorer = scorer_for(serving)
    if warmup:
        res = ModelWarmer(WarmupConfig(iterations=2)).warm(lambda p, n: serving.generate(p, timeout=120.0, max_tokens=n), w.config.vocab_size, ModelHealth())
        print(f"warm-up: {'ok' if res.success else 'FAILED ' + str(res.error)} ({res.total_ms:.0f} ms)", file=sys.stderr)
    return st


def cmd_serve(a) -> int:
    from .serving.api import serve
    st = build_app_state(None if a.demo else a.model, a.gpu, a.max_batch, a.max_seq_len, warmup=not a.no_warmup, kv_dtype=a.kv_dtype,
                         tp_comm=a.tp_comm, draft_layers=a.draft_layers, prefill_chunk=a.prefill_chunk)
    if a.classical:
        from .serving.classical import ClassicalModel, ClassicalServeState
        data = Path(a.classical).read_bytes()
        st.classical = ClassicalServeState(ClassicalModel.from_apr(data), data)
    print(f"serving '{st.model_name}' ({st.compute_mode}) on http://{a.host}:{a.port}", file=sys.stderr)
    try:
        serve(st, a.host, a.port)
    finally:
        if st.serving is not None:
            st.serving.stop()
            if hasattr(st.serving.engine, "shutdown"):
                st.serving.engine.shutdown()                  # tensor parallel: release the follower ranks
    return 0


def cmd_list(a) -> int:
    from .runtime.registry import list_local_models, model_home
    ms = list_local_models()
    if a.format == "json":
        print(json.dumps(ms))
    elif not ms:
        print(f"no models under {model_home()}")
    else:
        print(f"{'NAME':<48} {'FORMAT':<12} {'SIZE':>10}")
        for m in ms:
            print(f"{m['name']:<48} {m['format']:<12} {format_size(m['size_bytes']):>10}")
    return 0


def cmd_registry_offline(a) -> int:
    from .runtime.registry import model_home
    print(f"'{a.cmd} {a.model}': remote registries need a network; place the file under {model_home()} or pass a path", file=sys.stderr)
    return 2


BENCH_SUITES = ("quantize", "cpu_decode", "cpu_generate", "tokenizer", "cache", "decode", "gemv", "gemm", "attn")


def run_bench_suite(suite: str, model: str = "tiny-llama") -> list:
    import numpy as np
    from .utils.benchlib import BenchResult, DynamicSampler
    res = []
    if suite == "quantize":
        from . import quant
        x = np.random.default_rng(0).standard_normal(256 * 1024).astype(np.float32)
        for qt in ("Q4_K", "Q6_K", "Q8_0"):
            q = quant.QType[qt]
            def f():
                t = time.perf_counter(); quant.quantize(x, q); return 1e3 * (time.perf_counter() - t)
            res.append(BenchResult(f"quantize_{qt}_256k", "ms", DynamicSampler(5, 40).run(f)))
    elif suite == "cpu_decode":
        from .models.config import named_config
        from .models.cpu_model import CpuModel
        from .models.weights import synthetic_weights
        w = synthetic_weights(named_config(model), seed=0)
        m = CpuModel(w, 256)
        m.prefill([1, 2, 3, 4])
        pos = [4]
        def f():
            t = time.perf_counter(); m.forward(5, pos[0]); pos[0] = pos[0] + 1 if pos[0] < 250 else 4; return 1e3 * (time.perf_counter() - t)
        s = DynamicSampler(10, 200).run(f)
        res.append(BenchResult(f"cpu_decode_{model}_ms_per_token", "ms", s))
        res.append(BenchResult(f"cpu_decode_{model}_tok_per_s", "tok/s", [1e3 / v for v in s], higher_is_better=True))
    elif suite == "cpu_generate":
        # the CPU headline configuration: Q4_K_M weights of the named shape, 128 prompt tokens then 128 greedy tokens
        from .models.config import named_config
        from .models.cpu_model import CpuModel
        from .models.weights import synthetic_weights
        cfg = named_config(model)
        m = CpuModel(synthetic_weights(cfg, scheme="Q4_K_M", seed=0), 300)
        prompt = [int(x) for x in np.random.default_rng(0).integers(0, cfg.vocab_size, 128)]
        t0 = time.perf_counter()
        lg = m.prefill(prompt)                               # chunks of 32 tokens: one batched product per projection and chunk
        t1 = time.perf_counter()
        tok = int(np.argmax(lg))
        for i in range(128):
            lg = m.forward(tok, 128 + i)
            tok = int(np.argmax(lg))
        t2 = time.perf_counter()
        res.append(BenchResult(f"cpu_generate_{model}_prompt_tok_per_s", "tok/s", [128 / (t1 - t0)], higher_is_better=True))
        res.append(BenchResult(f"cpu_generate_{model}_decode_tok_per_s", "tok/s", [128 / (t2 - t1)], higher_is_better=True))
    elif suite == "tokenizer":
        from .serving.tokenizer import BPETokenizer, bytes_to_unicode
        b2u = bytes_to_unicode()
        tok = BPETokenizer([b2u[i] for i in range(256)] + ["Ġthe", "Ġquick", "Ġbrown", "Ġfox"], None)
        text = "the quick brown fox jumps over the lazy dog " * 64
        def f():
            t = time.perf_counter(); tok.encode(text); return 1e3 * (time.perf_counter() - t)
        res.append(BenchResult("tokenizer_encode_2.8kB", "ms", DynamicSampler(5, 50).run(f)))
    elif suite == "cache":
        from .runtime.paged_kv import PagedKvCache
        def f():
            c = PagedKvCache(4096, 16)
            t = time.perf_counter()
            for s in range(64):
                c.add_sequence(s); c.reserve(s, 512)
            for s in range(64):
                c.free_sequence(s)
            return 1e3 * (time.perf_counter() - t)
        res.append(BenchResult("paged_kv_open_reserve_close_64x512", "ms", DynamicSampler(5, 50).run(f)))
    elif suite in ("gemv", "gemm", "attn"):
        import subprocess
        out = subprocess.run([sys.executable, "-m", "realizar_b200.utils.kernel_bench", suite], capture_output=True, text=True, check=True).stdout
        d = json.loads(out.strip().splitlines()[-1])
        res.append(BenchResult(f"kernel_{suite}", "us", [d.get("us", d.get("ms", 0.0))], meta=d))
    elif suite == "decode":
        import subprocess
        out = subprocess.run([sys.executable, str(Path(__file__).resolve().parent.parent / "bench.py")], capture_output=True, text=True, check=True).stdout
        d = json.loads(out.strip().splitlines()[-1])
        res.append(BenchResult("decode_tok_per_s", d["unit"], [d["value"]], higher_is_better=True, meta=d))
    else:
        raise SystemExit(f"unknown suite '{suite}' (available: {', '.join(BENCH_SUITES)})")
    return res


def cmd_bench(a) -> int:
    from .utils.benchlib import save_results
    from .utils.stats import summarize
    if a.list or a.suite is None:
        print("\n".join(BENCH_SUITES))
        return 0
    res = run_bench_suite(a.suite, a.model)
    for r in res:
        s = summarize(r.samples)
        print(f"{r.name}: mean {s.mean:.4f} {r.unit} (n={s.n}, cv {100 * s.cv:.1f}%, p50 {s.p50:.4f}, p99 {s.p99:.4f})")
    if a.output:
        save_results(a.output, res)
    return 0


def cmd_bench_serving(a) -> int:
    from .utils.benchlib import convoy_test, saturation_test
    st = build_app_state(a.model, None, 4, 2048, warmup=a.model is not None)
    vocab = 100 if a.model is None else 1000
    r = convoy_test(st.serving, vocab=vocab) if a.cmd == "bench-convoy" else saturation_test(st.serving, a.concurrency, a.requests, vocab=vocab)
    st.serving.stop()
    print(json.dumps(r, indent=1))
    if a.output:
        Path(a.output).write_text(json.dumps(r))
    return 0 if r.get("ok", True) else 1


def cmd_bench_load(a) -> int:
    from .utils.loadgen import LoadConfig, run_load
    cfg = LoadConfig(a.requests, a.rate, a.concurrency, a.prompt_tokens, a.prompt_tokens_max, a.prompt_chars, a.max_tokens, a.temperature, a.top_p)
    if a.url:
        r = run_load(cfg, url=a.url)
    else:
        from .serving.api import create_app
        st = build_app_state(a.model, None, a.max_batch, a.max_seq_len, warmup=a.model is not None, tp_comm=a.tp_comm, prefill_chunk=a.prefill_chunk)
        try:
            app = create_app(st)
            if a.http:
                # a real listening socket: uvicorn on a local port in a thread of this process, the load goes through TCP + HTTP
                import threading
                import uvicorn
                server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=a.port, log_level="warning"))
                th = threading.Thread(target=server.run, daemon=True)
                th.start()
                t_end = time.time() + 30
                while not server.started and time.time() < t_end:
                    time.sleep(0.05)
                try:
                    r = run_load(cfg, url=f"http://127.0.0.1:{a.port}")
                finally:
                    server.should_exit = True
                    th.join(10)
                r["transport"] = "http"
            else:
                r = run_load(cfg, app=app)
                r["transport"] = "in-process ASGI"
            r["engine"] = st.serving.metrics()
        finally:
            st.serving.stop()
            if hasattr(st.serving.engine, "shutdown"):
                st.serving.engine.shutdown()                  # tensor parallel: release the follower ranks
    print(json.dumps(r, indent=1))
    if a.output:
        Path(a.output).write_text(json.dumps(r))
    return 0 if r["errors"] == 0 else 1


def cmd_bench_compare(a, strict: bool = False) -> int:
    from .utils.benchlib import compare_results, has_regression, load_results
    f1, f2 = (a.file1, a.file2) if hasattr(a, "file1") else (a.baseline, a.current)
    cmp = compare_results(load_results(f1), load_results(f2), 0.0 if strict and getattr(a, "strict", False) else getattr(a, "threshold", 5.0))
    for c in cmp:
        print(f"{c.name:<44} {c.baseline:>12.4f} -> {c.current:>12.4f}  {c.change_pct:+7.2f}%  p={c.p_value:.3g}  {c.verdict}")
    return 1 if strict and has_regression(cmp) else 0


def cmd_viz(a) -> int:
    import numpy as np
    from .utils.viz import full_report
    if a.file:
        from .utils.benchlib import load_results
        for r in load_results(a.file).values():
            print(full_report(r.name, r.samples, r.unit))
    else:
        print(full_report("demo latency", np.random.default_rng(0).lognormal(2.5, 0.3, a.samples), "ms"))
    return 0


def cmd_convert(a) -> int:
    from .formats.convert import convert
    print(json.dumps(convert(a.src, a.dst, to=a.to, qtype=a.qtype, compression=a.compression)))
    return 0


def cmd_monitor(a) -> int:
    from .utils.tui import run_monitor
    return run_monitor(a.url, a.interval, once=a.once)


def model_info(path: str) -> dict:
    from .formats.detect import detect_format, load_model, validate_weights
    from .quant import QType
    p = Path(path)
    w = load_model(p)
    c = w.config
    types: dict = {}
    nbytes = 0
    for t in w.tensors.values():
        qn = QType(t.qtype).name
        types[qn] = types.get(qn, 0) + 1
        nbytes += t.nbytes
    return {"path": str(p), "format": detect_format(p), "file_size": format_size(sum(f.stat().st_size for f in ([p] if p.is_file() else p.glob("*")))),
            "architecture": c.architecture, "hidden_dim": c.hidden_dim, "layers": c.num_layers, "heads": c.num_heads, "kv_heads": c.num_kv_heads,
            "head_dim": c.head_dim, "intermediate_dim": c.intermediate_dim, "vocab_size": c.vocab_size, "context_length": c.context_length,
            "rope_theta": c.rope_theta, "tensor_count": len(w.tensors), "tensor_types": types, "weight_bytes": nbytes, "validation": validate_weights(w)}


def cmd_info(a) -> int:
    import torch
    from . import __version__
    if a.model:
        print(json.dumps(model_info(a.model), indent=1, default=str))
        return 0
    print(f"realizar-b200 {__version__}")
    print(f"torch {torch.__version__}, cuda available: {torch.cuda.is_available()}")
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        print(f"device 0: {p.name}, sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.0f} GiB; {torch.cuda.device_count()} device(s)")
    from ._native import cpu_lib
    print(f"native CPU library: {cpu_lib()._name}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    table = {"run": cmd_run, "chat": cmd_chat, "serve": cmd_serve, "list": cmd_list, "pull": cmd_registry_offline, "push": cmd_registry_offline,
             "bench": cmd_bench, "bench-serving": cmd_bench_load, "bench-convoy": cmd_bench_serving, "bench-saturation": cmd_bench_serving, "bench-compare": cmd_bench_compare,
             "bench-regression": lambda x: cmd_bench_compare(x, strict=True), "viz": cmd_viz, "convert": cmd_convert, "monitor": cmd_monitor, "info": cmd_info}
    try:
        return table[a.cmd](a)
    except (FileNotFoundError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
