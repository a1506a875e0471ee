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
