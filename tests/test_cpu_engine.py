"""C++ CPU decoder against the fp32 oracle, and the host-side KV page manager."""
import numpy as np
import pytest

from realizar_b200.models.config import named_config
from realizar_b200.models.cpu_model import CpuModel
from realizar_b200.models.reference import ReferenceDecoder
from realizar_b200.models.weights import synthetic_weights
from realizar_b200.runtime.paged_kv import OutOfPages, PagedKvCache


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-phi2", "tiny-qwen2"])
def test_cpu_engine_matches_oracle(name):
    cfg = named_config(name)
    w = synthetic_weights(cfg, seed=1, std=0.05)
    ref, cpu = ReferenceDecoder(w), CpuModel(w, 64)
    toks = [3, 17, 200, 45, 9, 300, 12, 12, 5]
    lr, lc = ref.forward(toks)[-1].numpy(), cpu.prefill(toks)
    cos = float(lr @ lc / np.linalg.norm(lr) / np.linalg.norm(lc))
    assert cos > 0.99 and int(lr.argmax()) == int(lc.argmax())
    assert cpu.layer_trace().shape == (cfg.num_layers,) and np.all(cpu.layer_trace() > 0)


def test_cpu_generate_is_deterministic_and_bounded():
    w = synthetic_weights(named_config("tiny-llama"), seed=2, std=0.08)
    m = CpuModel(w, 32)
    a, tp, td = m.generate_greedy([1, 2, 3], 8)
    b, _, _ = CpuModel(w, 32).generate_greedy([1, 2, 3], 8)
    assert a == b and len(a) == 8 and tp > 0 and td > 0
    with pytest.raises(ValueError):
        m.generate_greedy([1] * 30, 8)
    with pytest.raises(ValueError):
        m.forward(10**6, 0)


def test_paged_kv_alloc_fork_prefix_and_rollback():
    kv = PagedKvCache(num_pages=8, page_size=16)
    kv.add_sequence(1)
    assert kv.reserve(1, 33) == kv.seqs[1].pages and len(kv.seqs[1].pages) == 3 and kv.free_page_count() == 5
    kv.fork(1, 2)
    assert kv.stats().shared_pages == 3
    page, copy_from = kv.ensure_writable(2, 2)
    assert copy_from == kv.seqs[1].pages[2] and page != copy_from and kv.refcount(copy_from) == 1
    kv.rollback(2, 16)
    assert len(kv.seqs[2].pages) == 1
    toks = list(range(40))
    kv.set_length(1, 33)
    assert kv.publish_prefix(1, toks) == 2
    kv.free_sequence(1); kv.free_sequence(2)
    kv.add_sequence(3)
    assert kv.match_prefix(3, toks) == 32 and len(kv.seqs[3].pages) == 2
    kv.add_sequence(4)
    assert kv.match_prefix(4, [99] + toks[1:]) == 0
    with pytest.raises(OutOfPages):
        kv.reserve(4, 16 * 9)


def test_chunked_prompt_pass_is_bit_identical_to_token_by_token():
    """The batched prompt pass (one batched product per projection and chunk, logits for the last token only) against feeding
    the prompt one token at a time: same logits bit for bit, also when the prompt is continued from a position, and the decode
    steps that follow agree."""
    import numpy as np
    from realizar_b200.models.config import named_config
    from realizar_b200.models.cpu_model import CpuModel
    from realizar_b200.models.weights import synthetic_weights
    for name in ("tiny-llama", "tiny-phi2", "tiny-qwen2"):
        cfg = named_config(name)
        w = synthetic_weights(cfg, scheme="Q4_K_M", seed=0)
        toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg.vocab_size, 45)]
        serial, la = CpuModel(w, 128), None
        for i, t in enumerate(toks):
            la = serial.forward(t, i)
        chunked = CpuModel(w, 128)
        lb = chunked.prefill(toks)
        split = CpuModel(w, 128)
        split.prefill(toks[:20], chunk=7)
        lc = split.prefill(toks[20:], pos0=20, chunk=16)
        assert np.array_equal(la, lb) and np.array_equal(la, lc), name
        assert np.array_equal(serial.forward(5, 45), chunked.forward(5, 45)), name
        with pytest.raises(ValueError):
            chunked.prefill([1] * 200)                         # past max_seq


def test_lock_step_decode_of_several_sequences_equals_separate_steps():
    """One batched step for three sequences (own KV caches, different lengths) against three single steps: same logits bit
    for bit over several steps; the CPU slot engine uses the lock-step path whenever more than one stream decodes."""
    import numpy as np
    from realizar_b200.models.config import named_config
    from realizar_b200.models.cpu_model import CpuModel
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.cpu_engine import CpuEngineConfig, CpuSlotEngine
    from realizar_b200.runtime.engine import SamplingParams
    for name in ("tiny-llama", "tiny-phi2"):
        w = synthetic_weights(named_config(name), scheme="Q4_K_M", seed=0)
        ms, ref = [CpuModel(w, 64) for _ in range(3)], [CpuModel(w, 64) for _ in range(3)]
        prompts = [[1, 2, 3, 4, 5], [9, 8, 7], [4, 4, 4, 4, 4, 4, 4]]
        for m, r, p in zip(ms, ref, prompts):
            m.prefill(p); r.prefill(p)
        toks, pos = [11, 12, 13], [len(p) for p in prompts]
        for _ in range(3):
            lg = CpuModel.forward_rows(ms, toks, pos)
            lr = np.stack([r.forward(t, p) for r, t, p in zip(ref, toks, pos)])
            assert np.array_equal(lg, lr), name
            toks, pos = [int(a.argmax()) for a in lg], [p + 1 for p in pos]
        with pytest.raises(ValueError):
            CpuModel.forward_rows([ms[0], ms[0]], [1, 2], [0, 0])      # the same handle twice
    eng = CpuSlotEngine(w, CpuEngineConfig(max_batch=3, max_seq_len=64))
    solo = CpuSlotEngine(w, CpuEngineConfig(max_batch=1, max_seq_len=64))
    firsts = {}
    for s, p in enumerate(prompts):
        eng.open_slot(s, 32); eng.set_sampling(s, SamplingParams(max_tokens=4))
        firsts[s] = eng.prefill(s, p)
    out = eng.feed(dict(firsts))
    for s, p in enumerate(prompts):
        solo.open_slot(0, 32); solo.set_sampling(0, SamplingParams(max_tokens=4))
        f = solo.prefill(0, p)
        assert f == firsts[s] and solo.feed({0: f})[0] == out[s]
        solo.close_slot(0)
