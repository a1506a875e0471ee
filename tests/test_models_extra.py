"""Grammar-constrained decoding, speculative decoding, MoE, Gated DeltaNet, encoder-decoder,
fp32 layers, classical-ML serving and explanations."""
import itertools
import json
import math

import numpy as np
import pytest
import torch

from realizar_b200.models import encoder_decoder as ED
from realizar_b200.models import layers as L
from realizar_b200.models import linear_attn as LA
from realizar_b200.models import moe as M
from realizar_b200.runtime import speculative as SP
from realizar_b200.serving import classical as C
from realizar_b200.serving import grammar as G


# -- grammar ------------------------------------------------------------------------------------------
def test_gbnf_parse_and_match():
    g = G.Grammar.from_gbnf('# answers\nroot ::= "yes" | "no" | num\nnum ::= "-"? [0-9]+ ("." [0-9]+)?\n')
    for ok in ("yes", "no", "12", "-3.25"):
        m = G.GrammarMatcher(g)
        assert m.advance(ok) and m.is_complete, ok
    m = G.GrammarMatcher(g)
    assert m.accepts("ye") and not m.accepts("yx") and m.advance("1.") and not m.is_complete and not m.advance("x")
    with pytest.raises(G.GrammarError):
        G.Grammar.from_gbnf('root ::= missing')
    with pytest.raises(G.GrammarError):
        G.Grammar.from_gbnf('other ::= "a"')
    esc = G.Grammar.from_gbnf(r'root ::= "a\n" [^\x00-\x1f"] "é"')
    mm = G.GrammarMatcher(esc)
    assert mm.advance("a\nzé") and mm.is_complete


def test_json_schema_grammar_and_token_mask():
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"type": "string"}},
                                                "kind": {"enum": ["a", "b"]}}, "required": ["name", "age", "tags", "kind"]}
    g = G.grammar_from_json_schema(schema)
    good = json.dumps({"name": "bob \"x\"", "age": -42, "tags": ["p", "q"], "kind": "b"})
    m = G.GrammarMatcher(g)
    assert m.advance(good) and m.is_complete
    for bad in ('{"name": 5', '{"age"', '{"name": "x", "age": 1.5', '{"name": "x", "age": 1, "tags": [], "kind": "c"'):
        assert not G.GrammarMatcher(g).advance(bad), bad
    vocab = ['{', '}', '"name"', ':', ' ', '"', 'bob', '42', ',', 'x', '{"name"', '<eos>']
    mk = G.GrammarTokenMasker(g, vocab, eos_token_id=11)
    allowed = {vocab[i] for i in np.nonzero(mk.mask())[0]}
    assert allowed == {'{', ' ', '{"name"'}
    assert mk.accept_token(10) and {vocab[i] for i in np.nonzero(mk.mask())[0]} == {':', ' '}
    logits = np.zeros(len(vocab))
    masked = mk.apply(logits)
    assert np.isinf(masked[vocab.index('bob')]) and masked[vocab.index(':')] == 0
    assert not mk.accept_token(11)          # EOS is not allowed mid-object


def test_constrained_generation_always_yields_valid_json():
    g = G.grammar_from_json_schema({"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}, "required": ["ok", "n"]})
    vocab = list('{}":,0123456789 -nokabc') + ['true', 'false', '"ok"', '"n"', 'null', 'abc', '<eos>']
    eos = len(vocab) - 1
    mk = G.GrammarTokenMasker(g, vocab, eos)
    rng = np.random.default_rng(0)
    text = ""
    for _ in range(200):
        x = mk.apply(rng.normal(size=len(vocab)))
        if mk.matcher.is_complete:
            x[eos] += 3.0                                  # bias towards stopping once a full object exists
        t = int(np.argmax(x))
        assert mk.accept_token(t)
        if t == eos:
            break
        text += vocab[t]
    obj = json.loads(text)
    assert isinstance(obj["ok"], bool) and isinstance(obj["n"], int)


def test_tool_calls():
    tools = [G.ToolDefinition("get_weather", "", {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}),
             G.ToolDefinition("add", "", {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}, "required": ["a", "b"]})]
    g = G.tool_call_grammar(tools)
    call = '{"name": "add", "arguments": {"a": 1.5, "b": 2}}'
    m = G.GrammarMatcher(g)
    assert m.advance(call) and m.is_complete
    assert not G.GrammarMatcher(g).advance('{"name": "rm"')
    tc = G.parse_tool_call("sure: " + call, tools)
    assert tc.name == "add" and tc.arguments == {"a": 1.5, "b": 2}
    assert G.parse_tool_call('{"name": "rm", "arguments": {}}', tools) is None and G.parse_tool_call("no json", tools) is None


# -- speculative ---------------------------------------------------------------------------------------
class _ToyModel:
    """Deterministic next-token function over the whole context (so drafts can disagree)."""

    def __init__(self, fn):
        self.fn, self.ctx = fn, []

    @property
    def position(self):
        return len(self.ctx)

    def forward(self, tokens):
        out = []
        for t in tokens:
            self.ctx.append(int(t))
            out.append(self.fn(self.ctx))
        return out

    def rollback(self, position):
        del self.ctx[position:]


def test_speculative_equals_target_greedy_for_any_draft():
    target_fn = lambda ctx: (sum(ctx) * 7 + len(ctx)) % 50
    ref_model = _ToyModel(target_fn)
    ref_model.forward([3, 4])
    ref, t = [], 5
    for _ in range(30):
        t = ref_model.forward([t])[0]
        ref.append(t)
    for name, draft_fn in (("same", target_fn), ("wrong", lambda c: 0), ("half", lambda c: target_fn(c) if len(c) % 2 else 1)):
        for k in (1, 3, 5):
            dec = SP.SpeculativeDecoder(_ToyModel(target_fn), _ToyModel(draft_fn), SP.SpeculativeConfig(k, 30))
            assert dec.generate([3, 4, 5]) == ref, (name, k)
            if name == "same":
                assert dec.stats.acceptance_rate == 1.0 and dec.stats.tokens_per_round > k * 0.8
            if name == "wrong":
                assert dec.stats.rounds >= 29
    # shared-cache (self-speculative) flavour: draft and target are the same object
    tm = _ToyModel(target_fn)
    dec = SP.SpeculativeDecoder(tm, tm, SP.SpeculativeConfig(4, 30), shared_cache=True)
    assert dec.generate([3, 4, 5]) == ref
    dec = SP.SpeculativeDecoder(_ToyModel(target_fn), _ToyModel(target_fn), SP.SpeculativeConfig(4, 30, eos_token_id=ref[7]))
    assert dec.generate([3, 4, 5]) == ref[:ref.index(ref[7]) + 1]
    ad = SP.SpeculativeDecoder(_ToyModel(target_fn), _ToyModel(target_fn), SP.SpeculativeConfig(2, 30, adaptive=True, max_k=6))
    assert ad.generate([3, 4, 5]) == ref and ad.stats.rounds < 10


def test_speculative_on_cpu_engine():
    from realizar_b200.models.config import named_config
    from realizar_b200.models.cpu_model import CpuModel
    from realizar_b200.models.weights import synthetic_weights
    w = synthetic_weights(named_config("tiny-llama"), seed=0, std=0.05)
    ref, _, _ = CpuModel(w, 128).generate_greedy([1, 2, 3, 4, 5], 16, None)
    d = SP.SpeculativeDecoder(SP.CpuSpecModel(CpuModel(w, 128)), SP.CpuSpecModel(CpuModel(w, 128)), SP.SpeculativeConfig(4, 16))
    assert d.generate([1, 2, 3, 4, 5]) == list(ref) and d.stats.rounds == 4


def test_rejection_sampling_preserves_target_distribution():
    rng = np.random.default_rng(0)
    p = np.array([[0.6, 0.3, 0.1], [0.2, 0.5, 0.3]])
    q = np.array([[0.2, 0.2, 0.6]])
    counts = np.zeros(3)
    for _ in range(20000):
        d = int(rng.choice(3, p=q[0]))
        counts[SP.rejection_sample([d], q, p, rng).tokens[0]] += 1
    assert np.abs(counts / counts.sum() - p[0]).max() < 0.015
    v = SP.verify_greedy([1, 2, 3], [1, 2, 9, 4])
    assert v.accepted == 2 and v.tokens == [1, 2, 9]
    assert SP.verify_greedy([1], [1, 5]).tokens == [1, 5]


# -- MoE ---------------------------------------------------------------------------------------------------
def test_moe_forward_matches_per_token_reference():
    w = M.MoeExpertWeights.random(8, 32, 64, shared_inter=48, seed=1)
    x = torch.randn(17, 32, generator=torch.Generator().manual_seed(0))
    assert (M.moe_forward(x, w, 2) - M.moe_forward_reference(x, w, 2)).abs().max() < 1e-5
    wts, idx = M.route_topk(x, w.router, 3)
    assert torch.allclose(wts.sum(-1), torch.ones(17)) and idx.shape == (17, 3)
    w2 = M.MoeExpertWeights.random(4, 16, 32)
    assert (M.moe_forward(x[:, :16], w2, 1, renormalize=False) - M.moe_forward_reference(x[:, :16], w2, 1, renormalize=False)).abs().max() < 1e-5


def test_moe_routers_and_controllers():
    r = M.CapacityFactorRouter(3, 2)
    picks = [r.route([0.9, 0.5, 0.1]) for _ in range(6)]
    assert picks == [0, 0, 1, 1, 2, 2]
    with pytest.raises(M.RouterError):
        r.route([1, 1, 1])
    r.release(0)
    assert r.route([0.9, 0.5, 0.1]) == 0
    with pytest.raises(M.RouterError):
        r.route([1.0])
    p2 = M.PowerOfTwoChoicesRouter(8, 1000, seed=0)
    for _ in range(4000):
        p2.route()
    assert max(p2.load) - min(p2.load) < 60          # far tighter than random assignment's spread
    h = M.HeijunkaController(100.0, 64)
    assert h.optimal_concurrency(200, 50) == 10 and h.should_shed(64, 10) and h.should_shed(5, 500) and not h.should_shed(5, 50)
    assert h.level(1000, 400)["shed"]
    pl = M.ExpertPlacement(4, hot_slots=1, warm_slots=1)
    pl.record([2, 2, 2, 0, 0, 3])
    t = pl.tiers()
    assert t[2] == M.ExpertTier.HOT and t[0] == M.ExpertTier.WARM and t[1] == M.ExpertTier.COLD


# -- linear attention -----------------------------------------------------------------------------------------
def test_gated_delta_rule():
    S = torch.zeros(1, 4, 3)
    k = LA.l2norm(torch.tensor([[1.0, 2.0, 0.5, -1.0]]), eps=0.0)
    v = torch.tensor([[0.3, -0.7, 2.0]])
    LA.gated_delta_step(S, k, k, v, torch.zeros(1), torch.ones(1))
    assert torch.allclose(torch.einsum("hkv,hk->hv", S, k), v, atol=1e-6)          # write then read returns the value
    v2 = torch.tensor([[1.0, 1.0, 1.0]])
    LA.gated_delta_step(S, k, k, v2, torch.zeros(1), torch.ones(1))
    assert torch.allclose(torch.einsum("hkv,hk->hv", S, k), v2, atol=1e-6)         # the delta rule overwrites, not accumulates
    S2 = S.clone()
    LA.gated_delta_step(S2, k, k, v2, torch.tensor([-1.0]), torch.zeros(1))
    assert torch.allclose(S2, S * math.exp(-1.0), atol=1e-6)                       # beta = 0: pure decay
    layer = LA.GatedDeltaNetLayer(32, LA.LinearAttnConfig(2, 8, 16))
    xs = torch.randn(6, 32, generator=torch.Generator().manual_seed(0))
    full, st = layer(xs)
    st2 = layer.new_state()
    a, _ = layer(xs[:4], st2)
    b, _ = layer(xs[4:], st2)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-6) and torch.allclose(st.S, st2.S)
    c = st.clone(); st.reset()
    assert c.S.abs().sum() > 0 and st.S.abs().sum() == 0
    state = torch.zeros(2, 3)
    w = torch.tensor([[1.0, 2.0, 3.0, 4.0], [0.0, 0.0, 0.0, 1.0]])
    ys = [LA.causal_conv1d_step(torch.tensor([float(t + 1), 1.0]), state, w) for t in range(4)]
    expect = torch.nn.functional.silu(torch.tensor([1 * 1 + 2 * 2 + 3 * 3 + 4 * 4.0, 1.0]))
    assert torch.allclose(ys[3], expect)


# -- encoder-decoder --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rel", [True, False])
def test_encoder_decoder_incremental_equals_full(rel):
    m = ED.EncoderDecoderModel(ED.EncDecConfig(use_rel_bias=rel), seed=3)
    src = torch.arange(2, 14)
    enc = m.encode(src)
    assert enc.shape == (12, 64)
    toks = [0, 5, 6, 7, 9]
    full, _ = m.decode(torch.tensor(toks), enc)
    cache, inc = None, []
    for t in toks:
        lg, cache = m.decode(torch.tensor([t]), enc, cache)
        inc.append(lg[0])
    assert (torch.stack(inc) - full).abs().max() < 1e-4 and cache.length == 5
    # encoder is bidirectional: changing the last source token changes the first encoder row
    src2 = src.clone(); src2[-1] = 99
    assert (m.encode(src2)[0] - enc[0]).abs().max() > 1e-4
    # decoder is causal: logits of position 0 do not depend on later tokens
    alt, _ = m.decode(torch.tensor([0, 8, 8, 8, 8]), enc)
    assert torch.allclose(alt[0], full[0], atol=1e-5)
    assert len(m.generate(src, 4)) <= 4


def test_t5_relative_buckets():
    rel = torch.arange(-200, 201)
    b = ED.relative_position_bucket(rel, True, 32, 128)
    assert b.min() == 0 and b.max() == 31 and b[200] == 0
    u = ED.relative_position_bucket(rel, False, 32, 128)
    assert (u[rel >= 0] == 0).all() and u[rel == -1] == 1 and u.max() == 31
    assert (torch.diff(u[rel <= 0].flip(0)) >= 0).all()


# -- fp32 layers ------------------------------------------------------------------------------------------------
def test_layers_incremental_and_fusions():
    torch.manual_seed(0)
    f = L.FusedLayerNormLinear(16, 8)
    f.norm.weight.data.normal_(); f.norm.bias.data.normal_()
    x = torch.randn(3, 16)
    assert (f(x) - f.linear(f.norm(x))).abs().max() < 1e-5
    yarn = L.RoPE(8, scaling=L.RopeScaling(L.RopeScalingType.YARN, 4.0, 16))
    for kw in ({}, {"kv_heads": 2, "rope": L.RoPE(8, neox=True)}, {"kv_heads": 1, "alibi": True}, {"window": 3, "fused_qkv": True, "rope": yarn}):
        a = L.Attention(32, 4, **kw)
        x = torch.randn(7, 32)
        full, _ = a(x)
        c, inc = None, []
        for t in range(7):
            o, c = a(x[t:t + 1], c)
            inc.append(o[0])
        assert (torch.stack(inc) - full).abs().max() < 1e-5, kw
    sw = L.SlidingWindowAttention(32, 4, window=2)
    x = torch.randn(6, 32)
    x2 = x.clone(); x2[0] += 5.0
    assert torch.allclose(sw(x)[0][5], sw(x2)[0][5], atol=1e-6) and not torch.allclose(sw(x)[0][1], sw(x2)[0][1])
    assert len(L.Model(50, 32, 4, 2, 64).generate([1, 2, 3], 4)) == 4


def test_rope_scaling_variants():
    base = L.RoPE(16).inv_freq()[0]
    lin = L.RoPE(16, scaling=L.RopeScaling(L.RopeScalingType.LINEAR, 4.0)).inv_freq()[0]
    assert torch.allclose(lin, base / 4)
    ntk = L.RoPE(16, scaling=L.RopeScaling(L.RopeScalingType.NTK, 4.0)).inv_freq()[0]
    assert torch.allclose(ntk[0], base[0]) and ntk[-1] < base[-1]
    dyn = L.RoPE(16, scaling=L.RopeScaling(L.RopeScalingType.DYNAMIC_NTK, 2.0, 128))
    assert torch.allclose(dyn.inv_freq(100)[0], base) and dyn.inv_freq(512)[0][-1] < base[-1]
    yarn, ms = L.RoPE(16, scaling=L.RopeScaling(L.RopeScalingType.YARN, 4.0, 64)).inv_freq()
    assert ms > 1.0 and torch.allclose(yarn[0], base[0]) and torch.allclose(yarn[-1], base[-1] / 4)
    q = torch.randn(5, 2, 16)
    for neox in (False, True):
        r = L.RoPE(16, neox=neox)
        out = r.apply(q, torch.arange(5))
        assert torch.allclose(out.norm(dim=-1), q.norm(dim=-1), atol=1e-5) and torch.allclose(out[0], q[0], atol=1e-6)
    part = L.RoPE(8).apply(q, torch.arange(5))
    assert torch.equal(part[..., 8:], q[..., 8:])
    assert torch.allclose(L.ALiBi(8).slopes, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    b = L.ALiBi(4).bias(2, 5)
    assert b.shape == (4, 2, 5) and b[0, 1, 4] == 0 and b[0, 0, 0] < 0


# -- classical ML ----------------------------------------------------------------------------------------------
def _toy_tree():
    return C.Tree(np.array([0, 1, -1, -1, 2, -1, -1]), np.array([0.5, 0.2, 0, 0, 0.7, 0, 0.]), np.array([1, 2, 0, 0, 5, 0, 0]),
                  np.array([4, 3, 0, 0, 6, 0, 0]), np.array([0, 0, 1., 3., 0, -2., 5.]), np.array([10, 6, 2, 4, 4, 1, 3.]))


def test_tree_shap_matches_brute_force_shapley():
    tr = _toy_tree()

    def cond(x, S, node=0):
        f = tr.feature[node]
        if f < 0:
            return tr.value[node]
        l, r = tr.left[node], tr.right[node]
        if f in S:
            return cond(x, S, l if x[f] <= tr.threshold[node] else r)
        return (tr.cover[l] * cond(x, S, l) + tr.cover[r] * cond(x, S, r)) / tr.cover[node]
    rng = np.random.default_rng(0)
    for _ in range(5):
        x = rng.random(3)
        phi = np.zeros(3)
        for i in range(3):
            others = [j for j in range(3) if j != i]
            for k in range(3):
                for S in itertools.combinations(others, k):
                    wgt = math.factorial(k) * math.factorial(3 - k - 1) / math.factorial(3)
                    phi[i] += wgt * (cond(x, set(S) | {i}) - cond(x, set(S)))
        assert np.allclose(C.tree_shap(tr, x), phi, atol=1e-9)


def test_classical_models_roundtrip_predict_explain():
    rng = np.random.default_rng(0)
    X = rng.normal(size=(6, 4))
    lin = C.ClassicalModel("LinearRegression", {"coef": rng.normal(size=(1, 4)), "intercept": np.array([0.5])}, feature_names=list("abcd"))
    lin2 = C.ClassicalModel.from_apr(lin.to_apr())
    assert np.allclose(lin2.predict(X), X @ lin.tensors["coef"][0] + 0.5, atol=1e-5) and lin2.feature_names == list("abcd")
    e = C.ShapExplainer(lin2, X.mean(0)).explain(X[0])
    assert e.verify_consistency(1e-4) and len(e.top_features(2)) == 2
    logit = C.ClassicalModel("LogisticRegression", {"coef": rng.normal(size=(3, 4)), "intercept": np.zeros(3)})
    P = logit.predict_proba(X)
    assert np.allclose(P.sum(1), 1) and (logit.predict(X) == P.argmax(1)).all()
    nb = C.ClassicalModel("NaiveBayes", {"theta": np.array([[0.0, 0, 0, 0], [3.0, 3, 3, 3]]), "var": np.ones((2, 4)), "class_prior": np.array([0.5, 0.5])})
    assert list(nb.predict(np.array([[0.1, 0, 0, 0], [2.9, 3, 3, 3]]))) == [0, 1]
    knn = C.ClassicalModel("KNN", {"X": np.array([[0.0, 0], [0, 1], [5, 5], [5, 6]]), "y": np.array([0, 0, 1, 1])}, {"k": 2, "n_classes": 2})
    assert list(knn.predict(np.array([[0.2, 0.2], [5, 5.5]]))) == [0, 1]
    km = C.ClassicalModel("KMeans", {"centers": np.array([[0.0, 0], [10, 10]])})
    assert list(km.predict(np.array([[1.0, 1], [9, 9]]))) == [0, 1]
    pca = C.ClassicalModel("PCA", {"mean": np.zeros(3), "components": np.eye(3)[:2]})
    assert pca.predict(np.array([[1.0, 2, 3]])).tolist() == [[1.0, 2.0]]
    tr = _toy_tree()
    forest = C.ClassicalModel("RandomForest", {**tr.to_tensors("tree.0"), **tr.to_tensors("tree.1")}, {"n_trees": 2, "task": "regression", "n_features": 3})
    f2 = C.ClassicalModel.from_apr(forest.to_apr())
    x = np.array([0.3, 0.9, 0.1])
    assert f2.predict(x[None])[0] == 3.0
    ex = C.ShapExplainer(f2).explain(x)
    assert ex.verify_consistency(1e-4) and abs(ex.base_value - 2.7) < 1e-5
    gb = C.ClassicalModel("GradientBoosting", tr.to_tensors("tree.0"), {"n_trees": 1, "learning_rate": 0.5, "init": 0.2, "n_features": 3})
    assert abs(gb.decision(x[None])[0] - (0.2 + 0.5 * 3.0)) < 1e-6 and C.ShapExplainer(gb).explain(x).verify_consistency(1e-4)
    with pytest.raises(C.ModelError):
        lin2.predict(np.zeros((1, 7)))
    with pytest.raises(C.ModelError):
        C.ShapExplainer(knn).explain(np.zeros(2))


def test_serve_state_audit_and_lambda(tmp_path):
    rng = np.random.default_rng(0)
    m = C.ClassicalModel("LogisticRegression", {"coef": rng.normal(size=(1, 4)), "intercept": np.array([0.3])})
    data = m.to_apr()
    sink = C.JsonFileAuditSink(str(tmp_path / "audit.jsonl"))
    st = C.ClassicalServeState(C.ClassicalModel.from_apr(data), data, sink=sink, background_mean=np.zeros(4), confidence_threshold=0.999)
    r = st.predict([0.1, 0.2, 0.3, 0.4], explain=True, client="alice")
    rec = sink.records()[0]
    assert rec["request_id"] == r["request_id"] and rec["input_dims"] == [4] and rec["nan_check_passed"] and rec["confidence_check_passed"] is False
    assert rec["warnings"] and rec["client_hash"] != "alice" and len(r["explanation"]["shap_values"]) == 4 and rec["latency_breakdown"]["explanation_ms"] is not None
    h = C.LambdaHandler(data)
    assert h.is_cold_start
    a, b = h.handle({"features": [1, 2, 3, 4]}), h.handle({"features": [1, 2, 3, 4]})
    assert a["cold_start"] and not b["cold_start"] and a["prediction"] == b["prediction"] and h.cold_start_ms > 0
    batch = h.handle_batch({"instances": [{"features": [1, 2, 3, 4]}, {"features": []}, {"features": [1, 2]}]})
    assert batch["success_count"] == 1 and batch["error_count"] == 2
    assert h.metrics.requests_failed == 2 and "lambda_requests_total 5" in h.metrics.to_prometheus()
    with pytest.raises(C.ModelError):
        C.LambdaHandler(b"")
    with pytest.raises(C.ModelError):
        C.LambdaHandler(b"GGUFxxxx")
    p = C.ProvenanceChain(training_data_hash="d", code_sha="c")
    p.add_distillation("teacher"); p.add_signature("me", "ed25519", "sig")
    assert p.distillation[0]["teacher_hash"] == "teacher" and p.signatures[0]["signer"] == "me"


def test_classical_http_endpoints():
    from fastapi.testclient import TestClient
    from realizar_b200.serving.api import AppState, create_app
    st = AppState.demo()
    try:
        c = TestClient(create_app(st))
        assert c.post("/v1/predict", json={"features": [1, 2]}).status_code == 501
        m = C.ClassicalModel("LinearRegression", {"coef": np.array([[2.0, -1.0]]), "intercept": np.array([0.5])})
        st.classical = C.ClassicalServeState(m)
        r = c.post("/v1/predict", json={"features": [1, 2]}).json()
        assert abs(r["prediction"] - 0.5) < 1e-6
        e = c.post("/v1/explain", json={"features": [1, 2]}).json()
        assert e["explanation"]["shap_values"] == [2.0, -2.0]
        assert c.get(f"/v1/audit/{e['request_id']}").json()["model_type"] == "LinearRegression"
        assert c.post("/v1/predict", json={"features": [1, 2, 3]}).status_code == 400
        assert c.post("/v1/predict", json={"features": "x"}).status_code == 400
        assert c.get("/v1/audit/none").status_code == 404
    finally:
        st.serving.stop()


def test_attention_over_ring_buffer_cache_equals_sliding_window():
    import torch
    from realizar_b200.models.layers import Attention, RoPE
    from realizar_b200.runtime.streaming_kv import StreamingKVCache
    torch.manual_seed(0)
    att = Attention(32, 4, kv_heads=2, rope=RoPE(8, 1e4), window=6)
    x = torch.randn(20, 32)
    with torch.no_grad():
        full, _ = att(x)                                        # whole sequence at once, window mask
        cache = StreamingKVCache(1, 6, 2, 8)
        ring = att.forward_streaming(x, cache)                  # token by token, six positions of memory
    assert cache.length[0] == 20 and cache.valid(0) == 6
    assert torch.allclose(full, ring, atol=1e-5)
    # with sink positions the first tokens stay visible: the result differs from the plain window once the ring has wrapped
    with torch.no_grad():
        sunk = att.forward_streaming(x, StreamingKVCache(1, 6, 2, 8, sinks=2))
    assert torch.allclose(full[:6], sunk[:6], atol=1e-5) and not torch.allclose(full[10:], sunk[10:], atol=1e-4)
