"""Scoring, per-request logit controls, speculative serving and the HTTP layer over a real GPU engine."""
import json
import math

import numpy as np
import pytest
import torch

from realizar_b200.models.config import ModelConfig, arch_constraints

pytestmark = pytest.mark.gpu


def _kq_llama():
    return ModelConfig("llama", 512, 2, 8, 2, 64, 1024, 512, 512, 1e4, 64, 0, 1e-5, 1, 2, arch_constraints("llama"))


@pytest.fixture(scope="module")
def engine_and_weights():
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = _kq_llama()
    w = synthetic_weights(cfg, scheme="Q4_K_M", seed=3, std=0.05)
    eng = DecodeEngine(w, EngineConfig(max_batch=4, max_seq_len=256, greedy_only=False))
    assert eng.gemm_ok
    return eng, w, cfg


def test_score_tokens_matches_fp32_oracle(cuda_device, engine_and_weights):
    """log p(token | prefix) from the tensor-core pass + log-softmax kernel against the fp32 reference decoder, for a prompt
    longer than the head plan's batch; perplexity and the pooled embedding come from the same pass."""
    from realizar_b200.models.reference import ReferenceDecoder
    eng, w, cfg = engine_and_weights
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg.vocab_size, 40)]
    out = eng.score_tokens(toks, want_embedding=True, top_k=3)
    ref_logits = ReferenceDecoder(w).forward(toks)                     # [T, V]
    ref_lp = torch.log_softmax(torch.as_tensor(np.asarray(ref_logits)), dim=-1)
    want = [float(ref_lp[i, toks[i + 1]]) for i in range(len(toks) - 1)]
    assert len(out["logprobs"]) == len(toks) - 1
    assert max(abs(a - b) for a, b in zip(out["logprobs"], want)) < 0.15
    assert abs(out["nll"] - (-sum(want) / len(want))) < 0.05 and abs(out["perplexity"] - math.exp(out["nll"])) < 1e-6
    assert len(out["embedding"]) == cfg.hidden_dim and all(math.isfinite(v) for v in out["embedding"])
    assert len(out["top_logprobs"]) == len(toks) - 1 and len(out["top_logprobs"][0]) == 3
    assert all(out["top_logprobs"][i][0][1] >= out["logprobs"][i] - 1e-4 for i in range(len(toks) - 1))   # nothing beats the top entry
    assert len(eng.free_slots()) == 4                                  # the scoring slot was released


def test_logit_controls_kernel_matches_reference(cuda_device):
    from realizar_b200 import ops
    B, V, W = 3, 1000, 16
    torch.manual_seed(0)
    logits = torch.randn(B, V, device="cuda") * 3
    hist = torch.full((B, W), -1, device="cuda", dtype=torch.int32)
    hist[0, :5] = torch.tensor([7, 7, 9, 400, 7], dtype=torch.int32)
    hist[1, :2] = torch.tensor([3, 999], dtype=torch.int32)
    rep = torch.tensor([1.5, 1.0, 1.2], device="cuda")
    pres = torch.tensor([0.25, 0.5, 0.0], device="cuda")
    freq = torch.tensor([0.1, 0.0, 0.0], device="cuda")
    bias = torch.zeros(B, V, device="cuda")
    bias[2, 10] = 5.0
    bias[2, 500:] = float("-inf")
    on = torch.tensor([0, 0, 1], device="cuda", dtype=torch.int32)
    want = logits.clone().cpu()
    want[2] += bias[2].cpu()
    for b in range(B):
        for tok in set(int(t) for t in hist[b].cpu() if t >= 0):
            cnt = int((hist[b] == tok).sum())
            v = float(want[b, tok])
            if float(rep[b]) != 1.0:
                v = v / float(rep[b]) if v > 0 else v * float(rep[b])
            want[b, tok] = v - float(pres[b]) - float(freq[b]) * cnt
    got = logits.clone()
    ops.logit_controls(got, hist, rep, pres, freq, bias, on)
    torch.cuda.synchronize()
    g, wv = got.cpu(), want
    assert torch.equal(torch.isinf(g), torch.isinf(wv)) and float((g[~torch.isinf(g)] - wv[~torch.isinf(wv)]).abs().max()) < 1e-5
    # history ring
    tokens = torch.tensor([11, 12, 13], device="cuda", dtype=torch.int32)
    pos = torch.tensor([17, -1, 3], device="cuda", dtype=torch.int32)
    ops.history_push(hist, tokens, pos, B)
    torch.cuda.synchronize()
    assert int(hist[0, 17 % W]) == 11 and int(hist[2, 3]) == 13 and int(hist[1, 2]) == -1


def test_engine_logit_bias_token_mask_and_penalties(cuda_device, engine_and_weights):
    """The controls act inside the captured sampling step: a token mask leaves one choice, a large logit_bias wins a greedy
    step, and a strong repetition penalty keeps a greedy stream from repeating a token within the history window."""
    from realizar_b200.runtime.engine import SamplingParams
    eng, w, cfg = engine_and_weights
    prompt = [3, 9, 27, 81, 243, 11, 5, 100, 7, 7, 19, 4]
    # mask: only token 123 allowed
    eng.open_slot(0, 64)
    eng.set_sampling(0, SamplingParams(temperature=0.8, top_k=40))
    allowed = np.zeros(cfg.vocab_size, dtype=bool)
    allowed[123] = True
    eng.set_token_mask(0, allowed)
    t = eng.prefill(0, prompt)
    assert t == 123
    assert int(eng.feed({0: t})[0]) == 123
    eng.set_token_mask(0, None)
    eng.close_slot(0)
    # logit_bias: +100 on token 77 under greedy decoding
    eng.open_slot(1, 64)
    eng.set_sampling(1, SamplingParams(temperature=0.0, logit_bias={77: 100.0}))
    assert eng.prefill(1, prompt) == 77 and int(eng.feed({1: 77})[1]) == 77
    eng.close_slot(1)
    # plain greedy for comparison, then with a strong repetition penalty: no token repeats inside the window
    outs = {}
    for name, sp in (("plain", SamplingParams(temperature=0.0, max_tokens=24)), ("rep", SamplingParams(temperature=0.0, max_tokens=24, repetition_penalty=50.0))):
        outs[name] = eng.generate(prompt, sp)
    assert len(set(outs["rep"])) == len(outs["rep"]) and not set(outs["rep"]) & set(prompt)
    assert eng.buf.bias_on.sum().item() == 0 and int((eng.buf.history >= 0).sum()) == 0        # everything was reset with the slots


def test_http_endpoints_over_gpu_engine_with_speculative_serving(cuda_device, engine_and_weights):
    """The OpenAI-style server over a real engine: scoring endpoints, a grammar-constrained and a stop-string completion,
    and self-speculative decoding for a lone greedy stream (same tokens as the engine's own greedy decoding, fewer passes)."""
    from starlette.testclient import TestClient
    from realizar_b200.runtime.engine import SamplingParams
    from realizar_b200.runtime.scheduler import SchedulerConfig, ServingEngine
    from realizar_b200.runtime.scorer import scorer_for
    from realizar_b200.serving.api import AppState, create_app
    from realizar_b200.serving.chat_template import RawTemplate
    from realizar_b200.serving.tokenizer import ByteTokenizer
    eng, w, cfg = engine_and_weights
    serving = ServingEngine(eng, SchedulerConfig(max_batch=4, max_seq_len=256), draft_layers=(0, 1), spec_k=3).start()
    st = AppState(serving, ByteTokenizer(256), RawTemplate(), "kq", None, compute_mode="gpu", context_length=256)
    st.scorer = scorer_for(serving)
    assert st.scorer is not None
    with TestClient(create_app(st)) as client:
        text = "the quick brown fox jumps over the lazy dog"
        lp = client.post("/v1/logprobs", json={"prompt": text}).json()
        assert len(lp["token_logprobs"]) == len(text) and lp["token_logprobs"][0] is None and all(v <= 0 for v in lp["token_logprobs"][1:])
        direct = eng_score = serving.call_on_engine(lambda e: e.score_tokens([ord(c) for c in text]))
        assert max(abs(a - b) for a, b in zip(lp["token_logprobs"][1:], direct["logprobs"])) < 1e-4
        pp = client.post("/v1/perplexity", json={"text": text}).json()
        assert abs(pp["nll"] - direct["nll"]) < 1e-4 and pp["perplexity"] > 1
        emb = client.post("/v1/embeddings", json={"input": [text, "abc"]}).json()
        assert len(emb["data"]) == 2 and len(emb["data"][0]["embedding"]) == cfg.hidden_dim
        body = {"model": "kq", "messages": [{"role": "user", "content": "hello world, hello"}], "max_tokens": 12, "temperature": 0}
        g = client.post("/v1/chat/completions", json={**body, "grammar": 'root ::= [ab]+'}).json()
        assert set(g["choices"][0]["message"]["content"]) <= set("ab") and len(g["choices"][0]["message"]["content"]) == 12
        # lone greedy stream: speculative rounds; the tokens are those of plain greedy decoding given their own prefix
        r = client.post("/v1/chat/completions", json={**body, "max_tokens": 24}).json()
        assert r["usage"]["completion_tokens"] == 24
        assert serving.spec_stats["rounds"] >= 1 and serving.spec_stats["drafted"] >= serving.spec_stats["accepted"]
        m = client.get("/metrics").text
        assert "realizar_requests_total" in m
    serving.stop()
    assert serving.health == "ok"
