"""GPU profile, memory pools, streaming plan, hybrid dispatch and the small batch / queue types."""
import pytest
import torch

from realizar_b200.runtime import batch_types as B
from realizar_b200.runtime import memory as M
from realizar_b200.runtime.gpu_profile import GpuProfile


def test_gpu_profile_env_overrides_and_policy():
    p = GpuProfile.detect(env={"RLZ_GEMV_STREAM": "1", "RLZ_PDL": "0", "RLZ_PREFILL_CHUNK": "256"})
    assert p.gemv_stream_variant and not p.pdl and p.prefill_chunk == 256 and p.cuda_graphs
    assert p.engine_config_overrides()["prefill_chunk"] == 256
    q = GpuProfile(sm_count=148, compute_capability=(10, 0))
    assert q.supported and q.gemv_target_ctas(1) == 296 and q.gemv_target_ctas(4) == 148
    assert q.attn_splits(32, 1) == 8 and q.attn_splits(8, 1) == 8 and q.attn_splits(32, 64) == 1 and q.attn_splits(2, 40) == 2
    assert not GpuProfile().supported and "gemm_decode_min_batch" in q.describe()


def test_memory_pools():
    assert M.size_class(1) == 256 and M.size_class(257) == 512 and M.size_class(4096) == 4096
    pool = M.GpuMemoryPool("cpu", max_pooled_bytes=2048)
    a = pool.acquire(300)
    assert a.numel() == 512 and pool.stats.bytes_in_use == 512
    pool.release(a)
    b = pool.acquire(400)
    assert b.data_ptr() == a.data_ptr() and pool.stats.hits == 1 and pool.stats.hit_rate == 0.5
    big = pool.acquire(4000)
    pool.release(big)                      # larger than the pooled-bytes cap: dropped
    pool.release(b)
    assert pool.stats.bytes_pooled == 512 and pool.trim() == 512 and not pool.free
    sp = M.StagingBufferPool(1024, 2)
    i0, b0 = sp.acquire()
    i1, _ = sp.acquire()
    assert sp.acquire() is None and b0.view(torch.float32, 4).numel() == 4
    sp.release(i0)
    assert sp.acquire()[0] == i0 and sp.mode in (M.TransferMode.PINNED, M.TransferMode.PAGEABLE)
    t = M.cache_aligned_empty(100, torch.float32, 64)
    assert t.data_ptr() % 64 == 0 and t.numel() == 100


def test_vram_check_and_layer_streamer():
    GB = 1 << 30
    c = M.check_vram_sufficient(40 * GB, 10 * GB, 180 * GB, 80)
    assert c.mode == M.StreamingMode.RESIDENT and c.resident_layers == 80
    c = M.check_vram_sufficient(400 * GB, 10 * GB, 180 * GB, 80)
    assert c.mode == M.StreamingMode.LAYER_STREAMING and 0 < c.resident_layers < 80 and c.layer_bytes == 5 * GB
    with pytest.raises(MemoryError):
        M.check_vram_sufficient(400 * GB, 175 * GB, 180 * GB, 80)
    log = []
    s = M.LayerStreamer(4, lambda l, b: log.append(("c", l, b)), lambda l, b: log.append(("x", l, b)), use_cuda=False)
    s.run()
    assert log == [("c", 0, 0), ("c", 1, 1), ("x", 0, 0), ("c", 2, 0), ("x", 1, 1), ("c", 3, 1), ("x", 2, 0), ("x", 3, 1)]


def test_hybrid_scheduler():
    h = M.HybridScheduler()
    assert h.choose(100) == M.ComputeBackend.CPU
    assert h.choose(1 << 20, operands_on_device=True) == M.ComputeBackend.GPU
    assert h.choose(1 << 20, operands_on_device=False) == M.ComputeBackend.GPU       # 6/20 of the CPU cost
    assert M.HybridScheduler(gpu_speedup=4.0).choose(1 << 20) == M.ComputeBackend.CPU  # transfer dominates
    assert M.HybridScheduler(gpu_available=False).choose(1 << 30) == M.ComputeBackend.CPU
    assert h.choose(10, preference=M.ComputeBackend.GPU) == M.ComputeBackend.GPU


def test_batch_and_queue_types():
    tb = B.TokenBatch(3)
    assert tb.push(1) is None and tb.push(2) is None and tb.push(3) == [1, 2, 3] and len(tb) == 0
    sb = B.SpeculativeBuffer(3)
    assert sb.add_candidate(5, 0.9) and sb.add_candidate(6, 0.8) and sb.add_candidate(7, 0.5) and not sb.add_candidate(8, 0.1)
    assert sb.verify([5, 6, 9]) == (2, 2) and sb.verify([5, 6, 7]) == (3, None)
    sb.accept(2)
    assert len(sb) == 1
    r = B.AsyncGpuResult()
    assert not r.is_ready()
    with pytest.raises(TimeoutError):
        r.wait(0.01)
    r.set_result(42)
    assert r.wait() == 42
    e = B.AsyncGpuResult(); e.set_error(ValueError("x"))
    with pytest.raises(ValueError):
        e.wait()
    q = B.AsyncRequestQueue(2)
    assert q.try_push(1) and q.try_push(2) and not q.try_push(3) and q.is_full and q.try_pop() == 1
    seen = []
    n = B.InferenceEventNotifier(); n.register(lambda *a: seen.append(a)); n.notify(1, 2.0, 3)
    assert seen == [(1, 2.0, 3)]
    m = B.InferenceMetrics(); [m.record(float(i), 2) for i in range(1, 101)]
    assert m.total_tokens == 200 and m.percentile(50) == 51.0 and m.percentile(99) == 100.0
    mb = B.MicroBatch(max_tokens=3)
    assert mb.add(B.BatchToken(1, 0, 0, True)) and mb.add(B.BatchToken(2, 0, 1, True)) and mb.add(B.BatchToken(9, 1, 5)) and not mb.add(B.BatchToken(0, 2, 0))
    assert (mb.num_prompt, mb.num_decode, mb.sequences()) == (2, 1, [0, 1])


def test_multi_request_policies_and_collector():
    s = B.MultiRequestScheduler(B.SchedulingPolicy.SJF, max_concurrent=1)
    a, b, c = s.submit(4, 10), s.submit(4, 2), s.submit(4, 5)
    order = []
    while not s.idle:
        for i in s.step():
            if i not in order:
                order.append(i)
    assert order == [b, c, a]
    f = B.MultiRequestScheduler(B.SchedulingPolicy.FCFS, max_concurrent=2)
    x, y, z = f.submit(1, 2), f.submit(1, 2), f.submit(1, 1)
    assert f.step() == [x, y] and f.step() == [x, y] and f.step() == [z] and f.idle
    rr = B.MultiRequestScheduler(B.SchedulingPolicy.ROUND_ROBIN, max_concurrent=2)
    p, q = rr.submit(1, 2), rr.submit(1, 2)
    assert [rr.step()[0] for _ in range(4)] == [p, q, p, q] and rr.idle
    now = [0.0]
    col = B.BatchRequestCollector(3, window_ms=5.0, clock=lambda: now[0])
    assert col.add("a") is None and col.poll() is None
    now[0] = 0.006
    assert col.poll() == ["a"]
    assert col.add(1) is None and col.add(2) is None and col.add(3) == [1, 2, 3]


def test_observability_primitives():
    from realizar_b200.utils.observability import ABTest, LatencyHistogram, Span, TraceContext
    c = TraceContext.new()
    p = TraceContext.from_traceparent(c.to_traceparent())
    assert p.trace_id == c.trace_id and p.parent_span_id == c.span_id and p.span_id != c.span_id and p.sampled
    for bad in ("", "00-abc-def-01", "01-" + "a" * 32 + "-" + "b" * 16 + "-01", "00-" + "0" * 32 + "-" + "b" * 16 + "-01", "00-" + "g" * 32 + "-" + "b" * 16 + "-01"):
        assert TraceContext.from_traceparent(bad) is None
    ch = c.child()
    assert ch.trace_id == c.trace_id and ch.parent_span_id == c.span_id
    s = Span("decode", c).set("tokens", 5).end()
    o = s.to_otel()
    assert o["name"] == "decode" and o["status"]["code"] == "ok" and s.duration_ms >= 0 and o["attributes"][0]["key"] == "tokens"
    h = LatencyHistogram()
    for ms in [1] * 50 + [20] * 45 + [400] * 4 + [99999]:
        h.observe(ms)
    assert h.percentile(50) == 1 and h.percentile(95) == 25 and h.percentile(99) == 500 and h.percentile(100) == float("inf")
    text = h.to_prometheus("ttft_seconds")
    assert 'ttft_seconds_bucket{le="+Inf"} 100' in text and "ttft_seconds_count 100" in text
    ab = ABTest("sampler", {"a": 1.0, "b": 3.0})
    picks = [ab.assign(f"user{i}") for i in range(4000)]
    assert ab.assign("user7") == ab.assign("user7") and 0.20 < picks.count("a") / 4000 < 0.30
    ab.record("a", 1.0); ab.record("a", 3.0)
    assert ab.summary()["a"] == {"n": 2, "mean": 2.0}


def test_streaming_kv_ring_buffer():
    from realizar_b200.runtime.streaming_kv import StreamingKVCache, StreamingKVCacheFp16
    c = StreamingKVCache(1, window=8, kv_heads=1, head_dim=2, sinks=2)
    for t in range(20):
        c.append(0, torch.full((1, 2), float(t)), torch.full((1, 2), -float(t)))
    k, v, pos = c.get(0)
    assert pos.tolist() == [0, 1, 14, 15, 16, 17, 18, 19] and k[:, 0, 0].tolist() == [0, 1, 14, 15, 16, 17, 18, 19] and v[-1, 0, 0] == -19
    assert c.valid(0) == 8 and c.length[0] == 20
    short = StreamingKVCache(2, window=8, kv_heads=1, head_dim=2)
    for t in range(3):
        short.append(1, torch.full((1, 2), float(t)), torch.zeros(1, 2))
    assert short.get(1)[2].tolist() == [0, 1, 2] and short.valid(0) == 0
    h = StreamingKVCacheFp16(1, 4, 2, 8)
    assert h.memory_bytes() == 2 * 4 * 2 * 8 * 2
    with pytest.raises(ValueError):
        StreamingKVCache(1, 2, 1, 2, sinks=2)


def test_step_program_builder_packs_ops_and_rejects_bad_programs():
    """Blob layout of the persistent decode-step program (CPU: the CUDA library is replaced by a stub)."""
    import ctypes
    import torch
    from realizar_b200.ops import _signatures as S
    from realizar_b200.ops.step_program import STEP_ARGMAX, STEP_ATTN, STEP_EMBED, STEP_GEMV, StepProgramBuilder

    class StubLib:
        def rlz_gemv_prepare(self, p, grid):
            q = ctypes.cast(p, ctypes.POINTER(S.GemvParams)).contents
            q.max_k, q.max_rows, q.any_generic = 2560, 61, 0
            ctypes.cast(grid, ctypes.POINTER(ctypes.c_int)).contents.value = 294
            return 0

        def rlz_gemv_smem_bytes(self, p):
            return 20000

        def rlz_decode_step_attn_smem(self, gt):
            return {1: 5000, 2: 8000, 4: 14000}.get(gt, -1)

    dev = torch.device("cpu")
    b = StepProgramBuilder(StubLib(), dev, occ=2, attn_gt=1, sm_count=148)
    assert b.grid == 296
    x = torch.zeros(2560)
    tok = torch.zeros(1, dtype=torch.int32)
    table = torch.zeros(1440 * 8, dtype=torch.uint8)
    b.add_embed(table, 12, 1440, 2560, 8, tok, x)
    g = S.GemvParams()
    g.batch, g.nmat = 1, 1
    b.add_gemv(g)
    a = S.AttnDecodeParams()
    a.n_heads, a.n_kv_heads, a.head_dim, a.splits, a.batch = 32, 32, 80, 8, 1
    b.add_attn(a)
    logits = torch.zeros(51200)
    out = torch.zeros(1, dtype=torch.int32)
    b.add_argmax(logits, 51200, out)
    prog = b.finish()
    assert prog.nops == 4 and prog.smem == 20000 and prog.params.occ == 2 and prog.params.attn_gt == 1
    raw = bytes(prog.blob.numpy())
    ops_tab = (S.StepOp * 4).from_buffer_copy(raw[: 4 * ctypes.sizeof(S.StepOp)])
    assert [o.kind for o in ops_tab] == [STEP_EMBED, STEP_GEMV, STEP_ATTN, STEP_ARGMAX]
    assert ops_tab[1].grid == 294 and ops_tab[2].grid == 32 * 8
    assert all(o.params % 16 == 0 for o in ops_tab) and ops_tab[0].params >= 4 * ctypes.sizeof(S.StepOp)
    emb = S.StepEmbed.from_buffer_copy(raw[ops_tab[0].params: ops_tab[0].params + ctypes.sizeof(S.StepEmbed)])
    assert emb.hidden == 2560 and emb.vocab == 8 and emb.row_bytes == 1440 and emb.out == x.data_ptr()
    gp = S.GemvParams.from_buffer_copy(raw[ops_tab[1].params: ops_tab[1].params + ctypes.sizeof(S.GemvParams)])
    assert gp.max_k == 2560 and gp.max_rows == 61          # the prepared copy is what travels, the caller's struct is untouched
    assert g.max_k == 0

    # argmax must end the program; batched or all-reduce GEMVs and int8 caches are refused
    b2 = StepProgramBuilder(StubLib(), dev, 1, 4, 148)
    b2.add_argmax(logits, 51200, out)
    b2.add_gemv(g)
    with pytest.raises(ValueError):
        b2.finish()
    g4 = S.GemvParams()
    g4.batch = 4
    with pytest.raises(ValueError):
        b2.add_gemv(g4)
    a.kv_q8 = 1
    with pytest.raises(ValueError):
        b2.add_attn(a)
    with pytest.raises(ValueError):
        StepProgramBuilder(StubLib(), dev, 1, 8, 148).add_attn(S.AttnDecodeParams(n_heads=8, n_kv_heads=1, splits=1, batch=1))


def test_guard_bands_name_the_overwritten_buffer():
    import torch
    from realizar_b200.runtime.memory import GuardBands
    g = GuardBands("cpu")
    a = g.zeros(5, 7, name="a")
    b = g.zeros(33, dtype=torch.int32, name="b")
    assert a.shape == (5, 7) and float(a.abs().sum()) == 0 and b.dtype == torch.int32
    a.fill_(3.0); b.fill_(-1)                                # writes inside the tensors leave the bands alone
    assert g.check() == []
    raw_b = g.entries[1][1]
    raw_b[GuardBands.BAND + 33 * 4] = 0                      # one byte past the end of b
    assert g.check() == ["b"]
    g.entries[0][1][GuardBands.BAND - 1] = 1                 # one byte before a
    assert g.check() == ["a", "b"] and g.bytes_reserved() >= 2 * 2 * GuardBands.BAND + 5 * 7 * 4 + 33 * 4


def test_layer_streaming_prefetch_order():
    """Which layer a streamed model starts copying when a layer is done: two places on in the pass's order (the next one already
    sits in the other buffer), wrapping into the next pass; nothing when at most two layers are streamed."""
    from realizar_b200.models.decoder import GpuModel
    m = object.__new__(GpuModel)
    m.streamed_from = 2
    order = list(range(7))                                   # layers 2..6 are streamed
    assert [m.prefetch_after(order, i) for i in range(7)] == [None, None, 4, 5, 6, 2, 3]
    assert [m.prefetch_after([0, 2, 4, 6], i) for i in range(4)] == [None, 6, 2, 4]          # a layer-skipping draft pass
    m.streamed_from = 5
    assert [m.prefetch_after(order, i) for i in range(7)] == [None] * 7                      # two streamed layers stay put
