"""Per-kernel micro-benchmarks with roofline fractions.

    python -m realizar_b200.utils.kernel_bench gemv --qtype Q4_K --n 200000 --k 2560 --batch 1
    python -m realizar_b200.utils.kernel_bench attn --heads 32 --kv-heads 32 --head-dim 80 --ctx 4096 --batch 8
    python -m realizar_b200.utils.kernel_bench gemm --qtype Q4_K --n 10240 --k 2560 --m 512
    python -m realizar_b200.utils.kernel_bench step-trace --model phi-2 --ctx 600
    python -m realizar_b200.utils.kernel_bench step-profile --model phi-2 --ctx 600

Each kernel is timed with CUDA events after warm-up.  Working sets are larger than the 126 MB
L2 (or rotated over several copies) so the numbers are DRAM numbers.  The achieved rate is
reported against the measured copy bandwidth / GEMM throughput of this machine when a
``MEASURED_PEAKS.json`` is present in the working directory, else against 6650 GB/s and
1590 TFLOP/s.  (Role of the reference's brick budgets, src/brick/mod.rs:47-442.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


def peaks():
    for p in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        if os.path.exists(p):
            d = json.load(open(p))
            return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


REPS = 1
GRAPH = False


def time_cuda(fn, iters: int, warmup: int = 3) -> float:
    """Median milliseconds per call over ``iters`` timed regions of ``REPS`` back-to-back calls
    (events on the current stream).  ``--reps`` > 1 amortises the launch and event overhead so the
    fixed cost of short kernels becomes visible (at the price of a warm L2 for small operands)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    run = None
    if GRAPH:                                   # replay the launches from a CUDA graph: no host launch cost in the timing
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(REPS):
                fn()
        run = g.replay
        run()
        torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if run is not None:
            run()
        else:
            for _ in range(REPS):
                fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / REPS)
    return float(np.median(times))


def random_weight(n: int, k: int, qtype, device):
    """Random valid blocks of ``qtype`` generated on the device, in the device layout."""
    from .. import ops
    from ..quant.torch_quant import quantize_torch
    step = max(1, (32 << 20) // k)
    parts = [quantize_torch(torch.randn(min(step, n - r), k, device=device) * 0.02, qtype) for r in range(0, n, step)]
    data = torch.cat(parts) if len(parts) > 1 else parts[0]
    return ops.upload_weight(data, qtype, n, k, device)


def bench_gemv(a):
    from .. import ops
    from ..quant import QType
    qt = QType[a.qtype]
    dev = torch.device("cuda")
    w = random_weight(a.n, a.k, qt, dev)
    x = torch.randn(a.batch, a.k, device=dev)
    y = torch.empty(a.batch, a.n, device=dev)
    g = torch.rand(a.k, device=dev) + 0.5
    xin = ops.VecIn(x, a.k, norm=ops.NORM_RMS if a.norm else ops.NORM_NONE, norm_w=g if a.norm else None)
    mats = [ops.MatOut([(w, 0)])]
    use_stream = ops.stream_eligible(mats) and not a.no_stream
    ar = None
    if a.ar:                                   # single-rank self-loop of the in-kernel all-reduce epilogue
        from ..parallel.tp import FusedTpComm
        comm = FusedTpComm(0, 1, dev)
        comm.allocate(1, a.n, max_batch=4)
        comm.begin_step()
        ar = comm.ar_desc(0)
    # --rotate R: R copies of the weights taken in turn, so that back-to-back launches stream from DRAM like the layers of a model
    ws = [w] + [random_weight(a.n, a.k, qt, dev) for _ in range(max(1, a.rotate) - 1)]
    ps = [ops.build_gemv_params([xin], [ops.MatOut([(wi, 0)])], y, a.batch, target_ctas=a.ctas or 148, ar=ar) for wi in ws]
    launch = ops.gemv_stream_launch if use_stream else ops.gemv_launch
    turn = [0]

    def run():
        launch(ps[turn[0] % len(ps)])
        turn[0] += 1
    ms = time_cuda(run, a.iters)
    byts = w.nbytes + x.numel() * 4 + y.numel() * 4
    pk = peaks()
    res = {"kernel": "gemv_stream" if use_stream else "gemv_slab" if ops.slab_eligible(ps[0]) else "gemv", "qtype": a.qtype, "n": a.n, "k": a.k, "batch": a.batch, "ms": ms, "bytes": byts,
           "gbs": byts / ms / 1e6, "frac_of_%s_hbm" % pk["source"]: byts / ms / 1e6 / pk["hbm_gbs"],
           "l2_note": "weights %.0f MB x %d %s L2" % (w.nbytes / 1e6, len(ws), ">" if w.nbytes * len(ws) > 126e6 else "<=")}
    if a.trace and not use_stream:
        res["phase_trace_us"] = gemv_phase_trace(lambda: time_cuda(run, 2, warmup=0), slab=ops.slab_eligible(ps[0]))
    return res


def gemv_phase_trace(run, slab: bool = False) -> dict:
    """Phase times of the last GEMV launch of ``run`` (medians over CTAs, microseconds)."""
    import ctypes
    from .. import ops
    lib = ops.lib()
    enable, read = (lib.rlz_gemv_slab_trace_enable, lib.rlz_gemv_slab_trace_read) if slab else (lib.rlz_gemv_trace_enable, lib.rlz_gemv_trace_read)
    n = 512
    buf = (ctypes.c_ulonglong * (n * 8))()
    ops.check(read(buf, n, 1), "gemv_trace_read")       # clear
    ops.check(enable(1), "gemv_trace_enable")
    torch.cuda.synchronize()
    run()
    torch.cuda.synchronize()
    ops.check(enable(0), "gemv_trace_enable")
    ops.check(read(buf, n, 0), "gemv_trace_read")
    t = np.frombuffer(buf, dtype=np.uint64).reshape(n, 8).astype(np.float64)
    t = t[t[:, 0] > 0]
    if not len(t):
        return {}
    names = {(0, 1): "prefetch_and_dependency_wait", (1, 2): "stage_input", (2, 3): "rows", (3, 6): "to_partial_sums", (6, 7): "epilogue"}
    out = {"ctas": int(len(t)), "span": float((t[:, 7].max() - t[:, 0].min()) / 1e3), "start_spread": float((t[:, 0].max() - t[:, 0].min()) / 1e3),
           "end_spread": float((t[:, 7].max() - t[:, 7].min()) / 1e3)}
    for (i, j), nm in names.items():
        ok = (t[:, i] > 0) & (t[:, j] > 0)
        if ok.any():
            d = t[ok, j] - t[ok, i]
            out[nm] = {"median": float(np.median(d) / 1e3), "max": float(d.max() / 1e3)}
    return out


def bench_attn(a):
    from .. import ops
    dev = torch.device("cuda")
    B, H, Hkv, d, ctx = a.batch, a.heads, a.kv_heads, a.head_dim, a.ctx
    pages_per_seq = -(-ctx // 16)
    n_pages = B * pages_per_seq
    kc = (torch.randn(n_pages, Hkv, 16, d, device=dev) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(n_pages, Hkv, 16, d, device=dev) * 0.5).to(torch.bfloat16)
    pt = torch.randperm(n_pages, device=dev).to(torch.int32).reshape(B, pages_per_seq).contiguous()
    qkv = torch.randn(B, (H + 2 * Hkv) * d, device=dev)
    out = torch.empty(B, H * d, device=dev)
    pos = torch.full((B,), ctx - 1, device=dev, dtype=torch.int32)
    splits = a.splits or max(1, min(32, (2 * 148) // (Hkv * B)))
    partial, counters = ops.attn_decode_scratch(B, H, splits, d, dev)
    p = ops.build_attn_decode_params(qkv, out, kc, vc, pos, pt, partial, counters, H, Hkv, d, splits, B, a.rope_dim, 2, 1e4, 0, H * d, (H + Hkv) * d)
    ms = time_cuda(lambda: ops.attn_decode_launch(p), a.iters)
    byts = 2 * B * ctx * Hkv * d * 2
    pk = peaks()
    return {"kernel": "attn_decode", "batch": B, "heads": H, "kv_heads": Hkv, "head_dim": d, "ctx": ctx, "splits": splits, "ms": ms,
            "kv_bytes": byts, "gbs": byts / ms / 1e6, "frac_of_%s_hbm" % pk["source"]: byts / ms / 1e6 / pk["hbm_gbs"],
            "l2_note": "KV %.0f MB %s L2" % (byts / 1e6, ">" if byts > 126e6 else "<=")}


def bench_prefill(a):
    """Causal prompt attention over the paged cache: ``--impl mma`` (16-query tiles, mma.sync) or ``tc`` (128-query tiles, tcgen05)."""
    os.environ["RLZ_PREFILL_ATT"] = a.impl                  # read once by the launcher, before the first launch
    from .. import ops
    dev = torch.device("cuda")
    H, Hkv, d, T = a.heads, a.kv_heads, a.head_dim, a.tokens
    pages = -(-T // 16)
    kc = (torch.randn(pages, Hkv, 16, d, device=dev) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(pages, Hkv, 16, d, device=dev) * 0.5).to(torch.bfloat16)
    pt = torch.randperm(pages, device=dev).to(torch.int32)
    qkv = torch.randn(T, (H + 2 * Hkv) * d, device=dev)
    out = torch.empty(T, H * d, device=dev, dtype=torch.bfloat16)
    ms = time_cuda(lambda: ops.attn_prefill(qkv, out, kc, vc, pt, T, 0, H, Hkv, d), a.iters)
    flops = 4.0 * H * d * T * (T + 1) / 2                   # QK^T and PV over the causal half
    pk = peaks()
    return {"kernel": "attn_prefill_" + a.impl, "tokens": T, "heads": H, "kv_heads": Hkv, "head_dim": d, "ms": ms, "tflops": flops / ms / 1e9,
            "frac_of_%s_bf16" % pk["source"]: flops / ms / 1e9 / pk["bf16_tflops"], "error": ops.attn_prefill_error()}


def bench_small(a):
    """The element-wise, norm, positional, cache-write and token-selection kernels at prompt-chunk / decode sizes, each timed
    alone: GB/s against the copy bandwidth (bytes = what the kernel has to read and write once)."""
    from .. import ops
    dev = torch.device("cuda")
    T, H, heads, d, V = a.tokens, a.hidden, a.heads, a.head_dim, a.vocab
    x = torch.randn(T, H, device=dev)
    xb = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    g, b = torch.rand(H, device=dev) + 0.5, torch.randn(H, device=dev) * 0.1
    qkv = torch.randn(T, 3 * heads * d, device=dev)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    table = ops.make_rope_table(T, a.rope_dim, 1e4, dev)
    pages = -(-T // 16)
    kc = torch.zeros(pages, heads, 16, d, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    rows = (pos // 16).to(torch.int32).contiguous()
    gate, up = torch.randn(T, 4 * H, device=dev), torch.randn(T, 4 * H, device=dev)
    act = torch.empty(T, 4 * H, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(a.batch, V, device=dev)
    temp, topk = torch.full((a.batch,), 0.7, device=dev), torch.full((a.batch,), 40, device=dev, dtype=torch.int32)
    topp, minp, uni = torch.full((a.batch,), 0.9, device=dev), torch.zeros(a.batch, device=dev), torch.rand(a.batch, device=dev)
    hist = torch.randint(0, V, (a.batch, 64), device=dev, dtype=torch.int32)
    ones, zeros = torch.full((a.batch,), 1.2, device=dev), torch.full((a.batch,), 0.1, device=dev)
    bias, on = torch.zeros(a.batch, V, device=dev), torch.ones(a.batch, device=dev, dtype=torch.int32)
    tgt = torch.randint(0, V, (a.batch,), device=dev, dtype=torch.int32)
    cases = {
        "norm_bf16 (LayerNorm -> bf16 operand)": (lambda: ops.norm_bf16(x, xb, g, b, ops.NORM_LAYER, 1e-5), T * H * 6),
        "rope_ (q and k heads, table)": (lambda: ops.rope_(qkv, pos, 2 * heads, d, a.rope_dim, 2, 1e4, table=table), T * 2 * heads * a.rope_dim * 8),
        "kv_append (bf16 pages)": (lambda: ops.kv_append(qkv[:, heads * d:], qkv[:, 2 * heads * d:], kc, vc, pos, rows, heads, d), T * 2 * heads * d * 6),
        "swiglu_bf16 (silu(gate) * up -> bf16)": (lambda: ops.swiglu_bf16(gate, up, act, ops.ACT_SILU), T * 4 * H * 10),
        "to_bf16": (lambda: ops.to_bf16(x, xb), T * H * 6),
        "argmax (%d x %d)" % (a.batch, V): (lambda: ops.argmax(logits), a.batch * V * 4),
        "sample top-k/top-p (%d x %d)" % (a.batch, V): (lambda: ops.sample(logits, temp, topk, topp, uni, minp), a.batch * V * 4),
        "logit_controls (bias row + penalties)": (lambda: ops.logit_controls(logits, hist, ones, zeros, zeros, bias, on), a.batch * V * 12),
        "logprob_parts (log-softmax pieces)": (lambda: ops.logprob_parts(logits, tgt), a.batch * V * 8),
    }
    pk = peaks()
    out = {"kernel": "small", "tokens": T, "hidden": H, "batch": a.batch, "vocab": V, "results": {}}
    for name, (fn, byts) in cases.items():
        if a.only and a.only not in name:
            continue
        ms = time_cuda(fn, a.iters)
        out["results"][name] = {"us": round(ms * 1e3, 2), "gbs": round(byts / ms / 1e6, 1), "frac_of_%s_hbm" % pk["source"]: round(byts / ms / 1e6 / pk["hbm_gbs"], 3)}
    return out


def bench_gemm(a):
    from ..ops import gemm as gemm_ops
    from ..quant import QType
    dev = torch.device("cuda")
    qt = QType[a.qtype]
    w = random_weight(a.n, a.k, qt, dev)
    x = (torch.randn(a.m, a.k, device=dev)).to(torch.bfloat16)
    y = torch.empty(a.m, a.n, device=dev, dtype=torch.float32)
    plan = gemm_ops.GemmPlan(w, a.m, dev, splitk=a.splitk or None, wide=a.wide)
    ms = time_cuda(lambda: plan.run(x, y), a.iters)
    trace = None
    if a.trace:
        trace = gemm_phase_trace(lambda: plan.run(x, y))
    flops = 2.0 * a.m * a.n * a.k
    pk = peaks()
    return {"kernel": "gemm_kquant_tcgen05", "qtype": a.qtype, "m": a.m, "n": a.n, "k": a.k, "wide": a.wide, "splitk": plan.splitk, "ms": ms, "tflops": flops / ms / 1e9,
            "frac_of_%s_bf16" % pk["source"]: flops / ms / 1e9 / pk["bf16_tflops"],
            "weight_gbs": w.nbytes / ms / 1e6, "frac_of_%s_hbm_weights" % pk["source"]: w.nbytes / ms / 1e6 / pk["hbm_gbs"],
            **({"phase_trace_us": trace} if trace else {})}


def gemm_phase_trace(run) -> dict:
    """Run one launch with the kernel's phase trace on; medians over CTAs of the time spent in each phase (microseconds)."""
    import ctypes
    import numpy as np
    from .. import ops
    lib = ops.lib()
    ops.check(lib.rlz_gemm_trace_enable(1), "gemm_trace_enable")
    torch.cuda.synchronize()
    run()
    torch.cuda.synchronize()
    ops.check(lib.rlz_gemm_trace_enable(0), "gemm_trace_enable")
    n = 1024
    buf = (ctypes.c_ulonglong * (n * 8))()
    ops.check(lib.rlz_gemm_trace_read(buf, n), "gemm_trace_read")
    t = np.frombuffer(buf, dtype=np.uint64).reshape(n, 8).astype(np.float64)
    t = t[t[:, 0] > 0]
    if not len(t):
        return {}
    names = ["setup", "dependency_wait", "first_weights", "k_loop", "mma_drain", "epilogue"]
    out = {"ctas": int(len(t)), "span": float((t[:, 6].max() - t[:, 0].min()) / 1e3),
           "start_spread": float((t[:, 0].max() - t[:, 0].min()) / 1e3)}
    for i, nm in enumerate(names):
        d = t[:, i + 1] - t[:, i]
        d = d[(t[:, i + 1] > 0) & (t[:, i] > 0)]
        if len(d):
            out[nm] = {"median": float(np.median(d) / 1e3), "max": float(d.max() / 1e3)}
    return out


def bench_step_trace(a):
    """Phase trace of the GEMV launches INSIDE the captured decode step of a named model shape (batch 1): one launch at a time is
    tagged, the step is replayed from its CUDA graph and the in-kernel time stamps of the tagged launch are read back.  Medians
    over CTAs in microseconds: dependency wait, input staging, warp 0's rows, epilogue; ``span`` = first entry to last exit."""
    import ctypes
    from .. import ops
    from ..models.config import named_config
    from ..models.weights import synthetic_weights
    from ..runtime.engine import DecodeEngine, EngineConfig
    cfg = named_config(a.model)
    # under torch.distributed.run the step is the tensor-parallel one: the epilogue of the row-parallel launches then holds
    # the in-kernel all-reduce (push to every peer, poll the own inbox), and the trace shows what it costs
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    comm = None
    if world > 1:
        import torch.distributed as dist
        from ..parallel.tp import make_tp_comm
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        comm = make_tp_comm(rank, world, torch.device("cuda", torch.cuda.current_device()), mode="fused")
    dev = torch.device("cuda", torch.cuda.current_device())
    eng = DecodeEngine(synthetic_weights(cfg, scheme="Q4_K_M", seed=0, device=dev), EngineConfig(max_batch=1, max_seq_len=a.ctx + 64, greedy_only=True),
                       device=dev, comm=comm, tp_rank=rank, tp_size=world)
    eng.open_slot(0, a.ctx + 32)
    eng.prefill(0, [int(t) for t in torch.randint(0, cfg.vocab_size, (a.ctx,), generator=torch.Generator().manual_seed(0))])   # same prompt on every rank
    plan = eng.plan(1)
    gemvs = [r[1] for r in plan.records if r and r[0] == "gemv"]
    per_layer = (len(gemvs) - 1) // cfg.num_layers
    lib, n = ops.lib(), 296
    buf = (ctypes.c_ulonglong * (n * 8))()
    out = {"kernel": "decode step phase trace", "model": a.model, "context": a.ctx, "gemv_launches": len(gemvs), "launches": {}}
    picks = [(per_layer * a.layer + i, f"layer {a.layer} gemv {i}") for i in range(per_layer)] + [(len(gemvs) - 1, "lm_head")]
    for which, name in picks:
        if not ops.slab_eligible(gemvs[which]):
            continue
        for p in gemvs:
            p._pad = 0
        gemvs[which]._pad = 1
        eng._graphs.clear()
        eng.buf.positions[:1].fill_(a.ctx)
        for _ in range(3):
            eng.run_step(1)
        torch.cuda.synchronize()
        lib.rlz_gemv_slab_trace_read(buf, n, 1)
        lib.rlz_gemv_slab_trace_enable(2)
        eng.run_step(1)
        torch.cuda.synchronize()
        lib.rlz_gemv_slab_trace_enable(0)
        lib.rlz_gemv_slab_trace_read(buf, n, 0)
        t = np.frombuffer(buf, dtype=np.uint64).reshape(n, 8).astype(np.int64)
        t = t[t[:, 0] > 0]
        med = lambda i, j: round(float(np.median(t[:, j] - t[:, i])) / 1e3, 2)
        out["launches"][name] = {"ctas": len(t), "wait": med(0, 1), "stage": med(1, 2), "rows_warp0": med(2, 3), "epilogue": med(6, 7),
                                 "epilogue_p90": round(float(np.percentile(t[:, 7] - t[:, 6], 90)) / 1e3, 2),
                                 "span": round(float(t[:, 7].max() - t[:, 0].min()) / 1e3, 2)}
    for p in gemvs:
        p._pad = 0
    out["world"] = world
    if world > 1:
        import torch.distributed as dist
        eng.close()
        comm.close()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return None
    return out


def bench_step_profile(a):
    """Per-launch CUDA-event times of the decode step of a named model shape, launch by launch without a graph (so without the
    overlap that programmatic dependent launch gives the captured step), plus the same step replayed from its graph, and the
    roofline budgets of the weight-streaming and attention launches."""
    from ..models.config import named_config
    from ..models.weights import synthetic_weights
    from ..runtime.engine import DecodeEngine, EngineConfig
    cfg = named_config(a.model)
    dev = torch.device("cuda")
    eng = DecodeEngine(synthetic_weights(cfg, scheme="Q4_K_M", seed=0, device=dev), EngineConfig(max_batch=max(a.batch, a.max_batch), max_seq_len=a.ctx + 192, greedy_only=True), device=dev)
    g = torch.Generator().manual_seed(0)
    for slot in range(a.batch):
        eng.open_slot(slot, a.ctx + 160)
        eng.prefill(slot, [int(t) for t in torch.randint(0, cfg.vocab_size, (a.ctx,), generator=g)])
    eng.buf.positions[:a.batch].fill_(a.ctx)
    rep = eng.brick_report(a.batch, steps=8)
    prof = eng.profile_step(a.batch, steps=8)
    for _ in range(3):
        eng.run_step(a.batch)
    eng.buf.positions[:a.batch].fill_(a.ctx)               # (rows whose position is -1 are idle: attention would skip them)
    ms = time_cuda(lambda: eng.run_step(a.batch), 20)
    return {"kernel": "decode step profile", "model": a.model, "batch": a.batch, "context": a.ctx, "graph_replay_us": round(1e3 * ms, 1),
            "eager_sum_us": round(rep["step_us"], 1), "launches": {k: {"per_step": v["count"] // 8, "avg_us": round(v["avg_us"], 2), "share": round(v["share"], 3)} for k, v in prof.items()},
            "budgets": {k: {"budget_us": round(v["budget_us"], 1), "gbs": None if v["gbs"] is None else round(v["gbs"], 1)} for k, v in rep["bricks"].items()},
            "bottleneck": rep["bottleneck"]}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reps", type=int, default=1, help="back-to-back launches per timed region")
    ap.add_argument("--graph", action="store_true", help="time a CUDA-graph replay of the launches")
    ap.add_argument("--pdl", action="store_true", help="launch with programmatic dependent launch")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("--qtype", default="Q4_K"); g.add_argument("--n", type=int, default=200000); g.add_argument("--k", type=int, default=2560)
    g.add_argument("--batch", type=int, default=1); g.add_argument("--iters", type=int, default=10); g.add_argument("--norm", action="store_true")
    g.add_argument("--ctas", type=int, default=0); g.add_argument("--no-stream", action="store_true"); g.add_argument("--ar", action="store_true")
    g.add_argument("--rotate", type=int, default=1, help="copies of the weights taken in turn (keeps back-to-back launches out of L2)")
    g.add_argument("--trace", action="store_true", help="add the kernel's per-phase times (medians over CTAs)")
    t = sub.add_parser("attn")
    t.add_argument("--heads", type=int, default=32); t.add_argument("--kv-heads", type=int, default=32); t.add_argument("--head-dim", type=int, default=80)
    t.add_argument("--ctx", type=int, default=4096); t.add_argument("--batch", type=int, default=8); t.add_argument("--splits", type=int, default=0)
    t.add_argument("--rope-dim", type=int, default=32); t.add_argument("--iters", type=int, default=10)
    pf = sub.add_parser("prefill")
    pf.add_argument("--impl", choices=["mma", "tc"], default="mma"); pf.add_argument("--tokens", type=int, default=512)
    pf.add_argument("--heads", type=int, default=32); pf.add_argument("--kv-heads", type=int, default=32); pf.add_argument("--head-dim", type=int, default=80)
    pf.add_argument("--iters", type=int, default=10)
    sm = sub.add_parser("small")
    sm.add_argument("--tokens", type=int, default=512); sm.add_argument("--hidden", type=int, default=2560); sm.add_argument("--heads", type=int, default=32)
    sm.add_argument("--head-dim", type=int, default=80); sm.add_argument("--rope-dim", type=int, default=32); sm.add_argument("--vocab", type=int, default=51200)
    sm.add_argument("--batch", type=int, default=64); sm.add_argument("--iters", type=int, default=10); sm.add_argument("--only", default="")
    m = sub.add_parser("gemm")
    m.add_argument("--qtype", default="Q4_K"); m.add_argument("--n", type=int, default=10240); m.add_argument("--k", type=int, default=2560)
    m.add_argument("--m", type=int, default=512); m.add_argument("--iters", type=int, default=10)
    m.add_argument("--splitk", type=int, default=0, help="0 = chosen from the shape")
    m.add_argument("--trace", action="store_true", help="add the kernel's per-phase times (medians over CTAs)")
    m.add_argument("--wide", type=int, default=0, help="0 auto, 1 force 128-row CTAs, 2 force 256-row CTAs (m > 128)")
    st = sub.add_parser("step-trace")
    st.add_argument("--model", default="phi-2"); st.add_argument("--ctx", type=int, default=600); st.add_argument("--layer", type=int, default=20)
    sp = sub.add_parser("step-profile")
    sp.add_argument("--model", default="phi-2"); sp.add_argument("--ctx", type=int, default=600); sp.add_argument("--batch", type=int, default=1)
    sp.add_argument("--max-batch", type=int, default=1, help="slots the engine is built for (buffer sizes)")
    a = ap.parse_args(argv)
    global REPS, GRAPH
    REPS, GRAPH = max(1, a.reps), a.graph
    if a.pdl:
        from .. import ops
        ops.set_pdl(True)
    res = {"gemv": bench_gemv, "attn": bench_attn, "gemm": bench_gemm, "prefill": bench_prefill, "small": bench_small, "step-trace": bench_step_trace, "step-profile": bench_step_profile}[a.cmd](a)
    if res is not None:
        print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
