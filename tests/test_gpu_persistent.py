"""The batch-1 decode step as one persistent cooperative kernel against the one-launch-per-operation plan."""
import numpy as np
import pytest
import torch

from realizar_b200.models.config import ModelConfig, arch_constraints, ROPE_NEOX

pytestmark = pytest.mark.gpu


def _phi2():
    return ModelConfig("phi2", 1280, 2, 16, 16, 80, 2560, 512, 512, 1e4, 32, ROPE_NEOX, 1e-5, None, 2,
                       arch_constraints("phi2"), parallel_residual=True, fused_qkv=True)


def _llama(kv_heads):
    return ModelConfig("llama", 512, 2, 8, kv_heads, 64, 1024, 512, 512, 1e4, 64, 0, 1e-5, 1, 2, arch_constraints("llama"))


def _cos(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("which,occ", [("phi2", 2), ("phi2", 1), ("llama-mha", 2), ("llama-g2", 1), ("llama-g4", 1)])
def test_persistent_step_matches_launch_per_op(cuda_device, monkeypatch, which, occ):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    cfg = {"phi2": _phi2, "llama-mha": lambda: _llama(8), "llama-g2": lambda: _llama(4), "llama-g4": lambda: _llama(2)}[which]()
    monkeypatch.setenv("RLZ_PERSIST_OCC", str(occ))
    w = synthetic_weights(cfg, seed=5, std=0.06)
    prompt = [3, 17, 200, 45, 9, 310, 77, 5, 120, 64, 33, 18, 250, 7, 91, 402, 11, 60, 29, 8, 300]
    # the same token sequence goes through both plans (the first plan's greedy choices), logits compared step by step:
    # free-running continuations could part at a near-tie between two logits without either plan being wrong
    forced, logits = None, []
    for persistent in (False, True):
        eng = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=256, greedy_only=True, persistent_step=persistent))
        eng.open_slot(0, 128)
        nxt = eng.prefill(0, prompt)
        fed, rows = [], []
        for i in range(40):
            tok = nxt if forced is None else forced[i]
            fed.append(tok)
            nxt = int(eng.feed({0: tok})[0])
            rows.append(eng.buf.logits[0, :cfg.vocab_size].float().cpu().numpy().copy())
        plan = eng.plan(1)
        assert (plan.program is not None) == persistent
        if persistent:
            assert plan.kernel_launches == 1
            plan.program.check()
        forced = forced or fed
        logits.append(rows)
        del eng
        torch.cuda.synchronize()
    worst = min(_cos(a, b) for a, b in zip(*logits))
    assert worst > 0.998, worst          # same GEMV code in both plans; the attention kernels differ (scalar vs tensor-core mode)
    agree = sum(int(a.argmax() == b.argmax()) for a, b in zip(*logits))
    assert agree >= 34, agree


def test_persistent_step_with_sampling_keeps_selection_kernel(cuda_device):
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    w = synthetic_weights(_phi2(), seed=2, std=0.06)
    eng = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=128, persistent_step=True))
    prompt = [1, 2, 3, 4, 5, 6, 7, 8]
    toks = eng.generate(prompt, SamplingParams(max_tokens=8, temperature=0.0))
    plan = eng.plan(1)
    assert plan.program is not None and plan.kernel_launches == 4      # step kernel + history update + logit controls + sampling kernel
    # every emitted token is an (almost) arg-max of the launch-per-operation plan's logits for the same prefix
    ref = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=128, persistent_step=False, greedy_only=True))
    ref.open_slot(0, 64)
    ref.prefill(0, prompt)
    for i, t in enumerate(toks):
        lg = ref.logits_of_last_step(0).float().cpu().numpy()[:ref.mcfg.vocab_size]
        assert lg[t] >= lg.max() - 0.12, (i, t)
        if i + 1 < len(toks):
            ref.feed({0: int(t)})
