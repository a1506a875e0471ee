"""End-to-end decode on the GPU against the fp32 oracle and the C++ CPU engine."""
import numpy as np
import pytest
import torch

from realizar_b200.models.config import ModelConfig, arch_constraints, named_config, ROPE_NEOX

pytestmark = pytest.mark.gpu


def small_phi2():
    return ModelConfig("phi2", 1280, 2, 16, 16, 80, 2560, 512, 512, 1e4, 32, ROPE_NEOX, 1e-5, None, 2,
                       arch_constraints("phi2"), parallel_residual=True, fused_qkv=True)


def _cos(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def near_greedy_violations(eng, prompt, out, tol=0.12, slot=3):
    """Teacher-force ``out`` after ``prompt`` through the single-token decode path and count the positions whose token is not
    an (almost) arg-max of that path's logits.  Two correct paths may break a near-tie differently and then continue
    differently; every token either of them emits must still be a near-arg-max given its own prefix."""
    vocab = eng.mcfg.vocab_size
    eng.open_slot(slot, len(prompt) + len(out) + 2)
    eng.cfg.batched_prefill_min, keep = 10 ** 9, eng.cfg.batched_prefill_min
    eng.prefill(slot, prompt)
    eng.cfg.batched_prefill_min = keep
    bad = 0
    for i, t in enumerate(out):
        lg = eng.logits_of_last_step(slot).float().cpu().numpy()[:vocab]
        bad += int(lg[t] < lg.max() - tol)
        if i + 1 < len(out):
            eng.feed({slot: int(t)})
    eng.close_slot(slot)
    return bad


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen2", "tiny-phi2", "small-phi2"])
@pytest.mark.parametrize("graphs", [False, True])
def test_engine_logits_match_oracle(cuda_device, name, graphs):
    from realizar_b200.models.reference import ReferenceDecoder
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = small_phi2() if name == "small-phi2" else named_config(name)
    w = synthetic_weights(cfg, seed=3, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, cuda_graphs=graphs, greedy_only=True))
    ref = ReferenceDecoder(w)
    toks = [5, 77, 300, 12, 9, 41, 200, 3, 3, 150, 88, 17, 400, 2, 61, 7, 19, 23]
    eng.open_slot(0, 64)
    nxt = eng.prefill(0, toks)
    got = eng.logits_of_last_step(0).cpu().numpy()
    want = ref.forward(toks)[-1].numpy()
    assert _cos(got, want) > 0.99, _cos(got, want)
    assert nxt == int(want.argmax()) or want[nxt] > np.sort(want)[-3]
    eng.close_slot(0)


def test_engine_matches_cpu_engine_tokens(cuda_device):
    from realizar_b200.models.cpu_model import CpuModel
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    cfg = named_config("tiny-llama")
    w = synthetic_weights(cfg, seed=11, std=0.08)
    eng = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=128, greedy_only=True))
    prompt = [1, 50, 60, 70, 80, 90]
    gpu = eng.generate(prompt, SamplingParams(max_tokens=12))
    cpu, _, _ = CpuModel(w, 128).generate_greedy(prompt, 12)
    agree = sum(int(a == b) for a, b in zip(gpu, cpu))
    assert agree >= 8, (gpu, cpu)          # both paths quantise activations differently; greedy paths rarely diverge


def test_engine_batch_slots_are_independent(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = named_config("tiny-llama")
    w = synthetic_weights(cfg, seed=4, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=4, max_seq_len=64, greedy_only=True))
    a, b = [3, 4, 5, 6, 7, 8], [100, 90, 80]
    eng.open_slot(0, 32)
    eng.prefill(0, a)
    la = eng.logits_of_last_step(0).cpu()
    eng.close_slot(0)
    # same prompts interleaved in different slots of a batched step
    eng.open_slot(1, 32); eng.open_slot(3, 32)
    for i in range(max(len(a), len(b))):
        feed = {}
        if i < len(a): feed[3] = a[i]
        if i < len(b): feed[1] = b[i]
        eng.feed(feed)
        if i == len(a) - 1:
            lb = eng.logits_of_last_step(3).cpu()
    assert float((la - lb).abs().max()) < 1e-3 * float(la.abs().max()) + 1e-5


def test_device_side_feedback_loop_matches_streaming(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    cfg = named_config("tiny-qwen2")
    w = synthetic_weights(cfg, seed=9, std=0.08)
    eng = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=64, greedy_only=True))
    prompt = [9, 8, 7, 6]
    streamed = eng.generate(prompt, SamplingParams(max_tokens=8))
    eng.open_slot(0, 32)
    first = eng.prefill(0, prompt)
    eng.buf.tokens[0] = first
    eng.buf.positions[0] = len(prompt)
    toks = [first]
    for _ in range(7):
        eng.run_step(1)
        eng.advance(1)
        toks.append(int(eng.buf.sampled[0]))
    assert toks == streamed


def _kq_llama():
    """A small Llama whose every projection is a K-quant (k % 256 == 0): the tensor-core prefill path."""
    from realizar_b200.models.config import ModelConfig, arch_constraints
    return ModelConfig("llama", 512, 2, 8, 2, 64, 1024, 512, 512, 1e4, 64, 0, 1e-5, 1, 2, arch_constraints("llama"))


@pytest.mark.parametrize("which", ["llama", "phi2", "llama-scaled-rope"])
def test_batched_prefill_matches_serial_and_oracle(cuda_device, which):
    import dataclasses
    from realizar_b200.models.reference import ReferenceDecoder
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = small_phi2() if which == "phi2" else _kq_llama()
    if which == "llama-scaled-rope":                  # linear context scaling: both paths must read the same (cos, sin) table
        cfg = dataclasses.replace(cfg, rope_scaling_type="linear", rope_scaling_factor=4.0)
    w = synthetic_weights(cfg, seed=7, std=0.05)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg.vocab_size, 77)]
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=256, greedy_only=True, prefill_chunk=32))
    assert eng.gemm_ok
    eng.open_slot(0, 128)
    nxt_b = eng.prefill(0, toks)                      # 3 tensor-core passes (32 + 32 + 13 tokens)
    lb = eng.logits_of_last_step(0).cpu().numpy()
    eng.close_slot(0)
    eng.cfg.batched_prefill_min = 10 ** 9             # force the token-by-token path
    eng.open_slot(1, 128)
    nxt_s = eng.prefill(1, toks)
    ls = eng.logits_of_last_step(1).cpu().numpy()
    assert _cos(lb, ls) > 0.995
    if which != "llama-scaled-rope":
        want = ReferenceDecoder(w).forward(toks)[-1].numpy()
        assert _cos(lb, want) > 0.99 and _cos(ls, want) > 0.99
    assert nxt_b == int(lb.argmax()) and nxt_s == int(ls.argmax())
    # decoding continues from a batched prefill exactly like from a serial one
    a = int(eng.feed({1: nxt_s})[1])
    eng.close_slot(1)
    eng.cfg.batched_prefill_min = 8
    eng.open_slot(0, 128)
    eng.prefill(0, toks)
    b = int(eng.feed({0: nxt_b})[0])
    assert nxt_b != nxt_s or a == b


@pytest.mark.parametrize("graphs", [False, True])
def test_tensor_core_decode_batch_matches_gemv_path(cuda_device, graphs):
    """A decode step of 16 sequences on the GEMM path gives the logits of the GEMV path."""
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = _kq_llama()
    w = synthetic_weights(cfg, seed=3, std=0.05)
    rng = np.random.default_rng(1)
    prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, 3 + (i % 5))] for i in range(16)]

    def run(min_batch, forced=None):
        """``forced``: the tokens to feed at each step (the other engine's choices), so that a near-tie between two logits
        cannot send the two engines down different continuations."""
        eng = DecodeEngine(w, EngineConfig(max_batch=16, max_seq_len=64, greedy_only=True, cuda_graphs=graphs, gemm_decode_min_batch=min_batch))
        for s, p in enumerate(prompts):
            eng.open_slot(s, 32)
            for t in p[:-1]:
                eng.feed({s: t})
        outs, fed = [], []
        last = {s: p[-1] for s, p in enumerate(prompts) if s != 5}          # slot 5 idles
        for i in range(3):
            if forced is not None:
                last = forced[i]
            fed.append(dict(last))
            got = eng.feed(last)
            outs.append(eng.buf.logits[:16, :cfg.vocab_size].float().cpu().numpy().copy())
            last = {s: int(got[s]) for s in last}
        return eng, outs, fed
    e_ref, ref, fed = run(10 ** 9)
    e_tc, tc, _ = run(16, forced=fed)
    assert e_tc._use_batched_step(16) and not e_ref._use_batched_step(16) and e_tc.kernels_per_step(16) > 0
    for a, b in zip(ref, tc):
        for s in range(16):
            if s != 5:
                assert _cos(a[s], b[s]) > 0.995, s


def test_forward_tokens_rollback_and_speculative(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    from realizar_b200.runtime.speculative import EngineSpecModel, LayerSkipDraft, SpeculativeConfig, SpeculativeDecoder
    cfg = _kq_llama()
    w = synthetic_weights(cfg, seed=5, std=0.05)
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, cfg.vocab_size, 9)]
    eng = DecodeEngine(w, EngineConfig(max_batch=4, max_seq_len=128, greedy_only=True))
    ref = eng.generate(prompt, SamplingParams(max_tokens=20))
    # one pass over several tokens gives the same next-token choices as token-by-token decoding
    # (compared through the decode path's logits for the same prefix: a near-tie may be broken differently by the two paths)
    prefix = prompt + ref[:6]
    eng.open_slot(2, 64)
    eng.cfg.batched_prefill_min, keep = 10 ** 9, eng.cfg.batched_prefill_min
    step_logits = []
    for t in prefix:
        eng.prefill(2, [t])
        step_logits.append(eng.logits_of_last_step(2).float().cpu().numpy()[:cfg.vocab_size].copy())
    eng.cfg.batched_prefill_min = keep
    eng.close_slot(2)
    eng.open_slot(0, 64)
    nxt = eng.forward_tokens(0, prefix)
    assert eng.slots[0].position == len(prompt) + 6
    for i in range(len(prompt) - 1, len(prefix)):
        assert step_logits[i][nxt[i]] >= step_logits[i].max() - 0.12, i
    assert sum(a == b for a, b in zip(nxt[len(prompt) - 1:], ref[:7])) >= 5
    # rollback then replay reproduces the continuation
    eng.rollback(0, len(prompt))
    again = eng.forward_tokens(0, ref[:3])[-1]
    assert step_logits[len(prompt) + 2][again] >= step_logits[len(prompt) + 2].max() - 0.12
    eng.close_slot(0)
    # draft = the target itself: every draft accepted, output identical to plain greedy decoding
    t, d = EngineSpecModel(eng, 0, 96), EngineSpecModel(eng, 1, 96)
    dec = SpeculativeDecoder(t, d, SpeculativeConfig(4, 20))
    out = dec.generate(prompt)
    # verification runs on the GEMM path, drafting on the GEMV path: a near-tie may flip and change the continuation, so the
    # output is checked token by token against the decode path's logits instead of against one fixed continuation
    assert len(out) == 20 and dec.stats.acceptance_rate >= 0.6 and dec.stats.rounds <= 10
    t.close(); d.close()
    assert near_greedy_violations(eng, prompt, out) == 0
    # self-speculative (layer-skipping draft over the shared cache): whatever is accepted, the output is the target's
    t = EngineSpecModel(eng, 0, 96)
    dec = SpeculativeDecoder(t, LayerSkipDraft(t), SpeculativeConfig(3, 20), shared_cache=True)
    out = dec.generate(prompt)
    assert len(out) == 20
    t.close()
    assert near_greedy_violations(eng, prompt, out) == 0


def test_prefix_cache_reuses_pages_and_parity_gate(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    cfg = _kq_llama()
    w = synthetic_weights(cfg, seed=9, std=0.05)
    rng = np.random.default_rng(4)
    shared = [int(t) for t in rng.integers(0, cfg.vocab_size, 40)]
    p1, p2 = shared + [5, 6, 7], shared + [9, 8]
    plain = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True, parity_gate=True))
    assert plain.parity_check(w) > 0.99
    want1, want2 = plain.generate(p1, SamplingParams(max_tokens=6)), plain.generate(p2, SamplingParams(max_tokens=6))
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True, prefix_cache=True))
    assert eng.generate(p1, SamplingParams(max_tokens=6)) == want1 and eng.prefix_hits == 0
    assert eng.generate(p2, SamplingParams(max_tokens=6)) == want2
    assert eng.prefix_hits == 1 and eng.prefix_tokens_reused == 32          # two full 16-token pages of the shared prefix
    assert eng.generate(p1, SamplingParams(max_tokens=6)) == want1 and eng.prefix_hits == 2
    assert eng.pages.stats().sequences == 0


def test_kv_snapshot_restore(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = _kq_llama()
    w = synthetic_weights(cfg, seed=13, std=0.05)
    toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg.vocab_size, 37)]
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True))
    eng.open_slot(0, 64)
    nxt = eng.prefill(0, toks)
    snap = eng.snapshot_kv(0)
    a = [int(eng.feed({0: nxt})[0])]
    a.append(int(eng.feed({0: a[-1]})[0]))
    eng.close_slot(0)
    eng.open_slot(1, 64)                     # other slot, other pages
    eng.restore_kv(1, snap)
    b = [int(eng.feed({1: nxt})[1])]
    b.append(int(eng.feed({1: b[-1]})[1]))
    assert snap["position"] == 37 and snap["pages"] == 3 and a == b


def test_engine_int8_kv_cache_tracks_bf16(cuda_device):
    """Decode and tensor-core prefill over the int8 KV cache stay close to the bf16 cache (same tokens early on,
    logits cosine > 0.995) and the cache takes (d + 16) / 2d of the memory."""
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = _kq_llama()
    w = synthetic_weights(cfg, seed=21, std=0.05)
    toks = [int(t) for t in np.random.default_rng(8).integers(0, cfg.vocab_size, 90)]
    res = {}
    for kd in ("bf16", "q8"):
        eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=160, greedy_only=True, kv_dtype=kd, prefill_chunk=64))
        eng.open_slot(0, 128)
        nxt = eng.prefill(0, toks)                            # flash prefill over the cache (two chunks)
        logits = [eng.logits_of_last_step(0).float().cpu().numpy()]
        out = [nxt]
        for _ in range(6):
            out.append(int(eng.feed({0: out[-1]})[0]))
            logits.append(eng.logits_of_last_step(0).float().cpu().numpy())
        res[kd] = (out, logits, eng.memory_report()["kv_bytes"])
    assert res["q8"][2] * 2 * 64 == res["bf16"][2] * (64 + 16)
    for a, b in zip(res["bf16"][1][:3], res["q8"][1][:3]):
        assert _cos(a, b) > 0.995
    assert res["bf16"][0][:2] == res["q8"][0][:2]


def test_profile_step_and_brick_report(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    w = synthetic_weights(small_phi2(), scheme="Q4_K_M", seed=1, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True))
    eng.open_slot(0, 64)
    eng.prefill(0, [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12])
    prof = eng.profile_step(1, steps=2)
    assert {"gemv", "attn"} <= set(prof) and abs(sum(v["share"] for v in prof.values()) - 1.0) < 1e-6
    assert prof["attn"]["count"] == 2 * small_phi2().num_layers
    rep = eng.brick_report(1, steps=2)
    assert rep["bottleneck"]["brick"] in rep["bricks"] and rep["step_us"] > 0
    assert rep["bricks"]["gemv"]["budget_us"] == pytest.approx(eng.model.weight_bytes() / (rep["bandwidth_gbs"] * 1e3 * 0.5))
    assert rep["bricks"]["attn"]["launches"] == small_phi2().num_layers


@pytest.mark.parametrize("scheme", ["Q4_0", "Q8_0", "Q5_0", "Q4_1", "F16", "BF16"])
def test_other_weight_types_run_prompts_on_the_tensor_core_path(cuda_device, scheme):
    """Checkpoints in the 32-weight block types and dense 16-bit checkpoints: every projection is eligible for the tcgen05 GEMM,
    so a prompt goes through the token-batch path (not token by token), and both paths agree with the fp32 oracle."""
    from realizar_b200.models.reference import ReferenceDecoder
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    from realizar_b200 import ops
    cfg = _kq_llama()
    w = synthetic_weights(cfg, scheme=scheme, seed=3, std=0.05)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg.vocab_size, 45)]
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True))
    assert eng.gemm_ok
    eng.open_slot(0, 96)
    before = ops.launch_count()
    eng.prefill(0, toks)
    batched_launches = ops.launch_count() - before
    lb = eng.logits_of_last_step(0).cpu().numpy()
    eng.cfg.batched_prefill_min = 10 ** 9             # the same prompt token by token through the decode kernels
    eng.open_slot(1, 96)
    eng.prefill(1, toks)
    assert batched_launches < len(toks)               # one pass over the 45 tokens, not 45 decode steps
    ls = eng.logits_of_last_step(1).cpu().numpy()
    want = ReferenceDecoder(w).forward(toks)[-1].numpy()
    assert _cos(lb, want) > 0.99 and _cos(ls, want) > 0.99 and _cos(lb, ls) > 0.995
    assert ops.device_error() == 0
    out = eng.feed({0: int(lb.argmax())})
    assert 0 <= int(out[0]) < cfg.vocab_size


def test_canaries_and_index_guards(cuda_device):
    """Guard bands around the step buffers stay intact over prompt passes and decode steps and a damaged band is reported; device
    indices outside their range are skipped and recorded (no access is made with them)."""
    from realizar_b200 import ops
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    w = synthetic_weights(_kq_llama(), seed=2, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=4, max_seq_len=128, canaries=True))
    assert eng.guards is not None and len(eng.guards.entries) > 10
    eng.generate([(5 * i + 1) % 500 for i in range(40)], SamplingParams(max_tokens=12, temperature=0.8, top_k=20))
    eng.generate([1, 2, 3], SamplingParams(max_tokens=4))
    eng.check_health()                                       # nothing wrote outside its buffer
    name, raw, nbytes = eng.guards.entries[3]
    raw[eng.guards.BAND + nbytes + 5] = 0                    # damage one band from the host
    with pytest.raises(ops.KernelError, match="guard bands"):
        eng.check_health()
    raw[eng.guards.BAND + nbytes + 5] = eng.guards.PATTERN
    eng.check_health()
    # index guards
    assert ops.device_error() == 0
    H, V = 64, 100
    table = torch.randn(V, H, device="cuda")
    out = torch.full((3, H), 7.0, device="cuda")
    toks = torch.tensor([5, 1000, -2], device="cuda", dtype=torch.int32)
    ops.embed(table.view(torch.uint8).reshape(V, -1), 0, H * 4, H, V, toks, out, None, None)
    torch.cuda.synchronize()
    assert torch.equal(out[0], table[5]) and float(out[1:].abs().sum()) == 0 and ops.device_error() == 3401       # (-2 marks an idle row: zeros, no error)
    kc = torch.zeros(4, 2, 16, 8, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kv = torch.randn(2, 2 * 8, device="cuda")
    pos = torch.tensor([3, 20], device="cuda", dtype=torch.int32)
    ops.kv_append(kv, kv, kc, vc, pos, torch.tensor([1, 9], device="cuda", dtype=torch.int32), 2, 8)     # page 9 of a 4-page cache
    torch.cuda.synchronize()
    assert float(kc[1].abs().sum()) > 0 and ops.device_error() == 3402
    pt = torch.zeros(2, 3, device="cuda", dtype=torch.int32)
    rows = torch.zeros(2, device="cuda", dtype=torch.int32)
    ops.page_rows(pt, torch.tensor([10, 100], device="cuda", dtype=torch.int32), rows, 2, 16)            # position 100 needs page-table column 6 of 3
    torch.cuda.synchronize()
    assert rows.tolist() == [0, -1] and ops.device_error() == 3403


@pytest.mark.parametrize("which", ["llama", "phi2"])
def test_layer_streaming_matches_resident_engine(cuda_device, which):
    """Only the first layer's matrices stay on the device; the other four are streamed from pinned host memory through two
    buffers (prompt pass on the tensor-core path, decode steps on the GEMV path, a layer-skipping draft step): same tokens and
    logits as the engine that keeps everything resident."""
    import dataclasses
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    cfg = dataclasses.replace(_kq_llama() if which == "llama" else small_phi2(), num_layers=5)
    w = synthetic_weights(cfg, seed=4, std=0.05)
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, cfg.vocab_size, 37)]
    outs, logits = [], []
    for resident in (None, 1):
        eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True, resident_layers=resident))
        assert eng.model.streaming == (resident is not None)
        outs.append(eng.generate(prompt, SamplingParams(max_tokens=10)))
        eng.open_slot(0, 64)
        eng.prefill(0, prompt[:9])
        eng.draft_step(0, 5, (0, 2, 4))                     # a pass over a subset of the layers
        eng.feed({0: 7})
        logits.append(eng.logits_of_last_step(0).float().cpu().numpy())
        eng.check_health()
        if resident is not None:
            assert eng.model.stream_copies > 4 * 10          # the four streamed layers were copied in every pass
            assert not eng.cfg.cuda_graphs
        eng.close()
        del eng
        torch.cuda.synchronize()
    assert outs[0] == outs[1], outs
    assert _cos(logits[0], logits[1]) > 0.9999


def test_engine_reset_returns_to_the_post_load_state(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    w = synthetic_weights(_kq_llama(), seed=2, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=128, greedy_only=True))
    first = eng.generate([1, 2, 3, 4, 5, 6, 7, 8, 9], SamplingParams(max_tokens=6))
    eng.open_slot(0, 64); eng.open_slot(1, 64)
    eng.prefill(0, [5, 6, 7]); eng.prefill(1, [9] * 20)
    used = eng.pages.stats().utilization
    assert used > 0 and len(eng.free_slots()) == 0
    eng.reset()
    assert len(eng.free_slots()) == 2 and eng.pages.stats().utilization == 0
    assert int(eng.buf.positions.max()) == -1
    assert eng.generate([1, 2, 3, 4, 5, 6, 7, 8, 9], SamplingParams(max_tokens=6)) == first
