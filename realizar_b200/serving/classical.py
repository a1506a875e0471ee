"""Classical-ML model serving from ``.apr`` files: ten estimator families restated as vectorised
numpy predictors, SHAP explanations (closed form for linear models, TreeSHAP for tree ensembles),
audit records with provenance, and a Lambda-style single-call handler with cold-start metrics.

An ``.apr`` classical model is an APR v2 file whose metadata carries ``model_type`` (one of
``MODEL_TYPES``) and estimator hyper-parameters, and whose tensors are the fitted arrays named
below.  Reference parity: ``LoadedModel`` / ``ServeState`` (src/serve.rs:86-427), APR model type
ids (src/model_loader.rs:293-310), ``ShapExplainer`` / ``DecisionTree`` (src/explain.rs:32-249),
``AuditRecord`` / sinks / ``ProvenanceChain`` (src/audit.rs:37-429), ``LambdaHandler`` (src/lambda.rs:39-439)."""
from __future__ import annotations

import hashlib
import json
import time
import uuid
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

MODEL_TYPES = {0x0001: "LinearRegression", 0x0002: "LogisticRegression", 0x0003: "DecisionTree", 0x0004: "RandomForest",
               0x0005: "GradientBoosting", 0x0006: "KMeans", 0x0007: "PCA", 0x0008: "NaiveBayes", 0x0009: "KNN", 0x000A: "SVM",
               0x0010: "NgramLM", 0x0011: "TFIDF", 0x0012: "CountVectorizer", 0x0020: "NeuralSequential", 0x0021: "NeuralCustom",
               0x0030: "ContentRecommender", 0x0040: "MixtureOfExperts", 0x00FF: "Custom"}
TYPE_IDS = {v: k for k, v in MODEL_TYPES.items()}


class ModelError(ValueError):
    pass


def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


@dataclass
class Tree:
    """Array-form binary tree: ``feature[i] < 0`` marks a leaf; go left when ``x[feature] <= threshold``."""
    feature: np.ndarray
    threshold: np.ndarray
    left: np.ndarray
    right: np.ndarray
    value: np.ndarray                   # [nodes] or [nodes, classes]
    cover: Optional[np.ndarray] = None  # training samples per node (TreeSHAP weights)

    def leaf_of(self, X: np.ndarray) -> np.ndarray:
        node = np.zeros(X.shape[0], dtype=np.int64)
        active = self.feature[node] >= 0
        while active.any():
            idx = np.nonzero(active)[0]
            n = node[idx]
            go_left = X[idx, self.feature[n]] <= self.threshold[n]
            node[idx] = np.where(go_left, self.left[n], self.right[n])
            active = self.feature[node] >= 0
        return node

    def predict_value(self, X: np.ndarray) -> np.ndarray:
        return self.value[self.leaf_of(X)]

    def to_tensors(self, prefix: str) -> Dict[str, np.ndarray]:
        d = {f"{prefix}.feature": self.feature.astype(np.int32), f"{prefix}.threshold": self.threshold.astype(np.float32),
             f"{prefix}.left": self.left.astype(np.int32), f"{prefix}.right": self.right.astype(np.int32), f"{prefix}.value": self.value.astype(np.float32)}
        if self.cover is not None:
            d[f"{prefix}.cover"] = self.cover.astype(np.float32)
        return d

    @classmethod
    def from_tensors(cls, t: Dict[str, np.ndarray], prefix: str) -> "Tree":
        g = lambda k: np.asarray(t[f"{prefix}.{k}"])
        return cls(g("feature").astype(np.int64), g("threshold").astype(np.float64), g("left").astype(np.int64), g("right").astype(np.int64),
                   g("value").astype(np.float64), np.asarray(t[f"{prefix}.cover"], np.float64) if f"{prefix}.cover" in t else None)


@dataclass
class ClassicalModel:
    model_type: str
    tensors: Dict[str, np.ndarray]
    params: Dict[str, Any] = field(default_factory=dict)
    feature_names: Optional[List[str]] = None

    # -- persistence ----------------------------------------------------------------------------
    def to_apr(self) -> bytes:
        from ..formats.apr import AprBuilder
        b = AprBuilder({"model_type": self.model_type, "model_type_id": TYPE_IDS[self.model_type], "params": self.params,
                        "feature_names": self.feature_names, "classical": True})
        for k, v in self.tensors.items():
            a = np.ascontiguousarray(np.asarray(v), dtype=np.float32)
            b.add_tensor_raw(k, a.shape or (1,), 0, a)
        return b.build()

    @classmethod
    def from_apr(cls, data) -> "ClassicalModel":
        from ..formats.apr import AprModel
        m = AprModel.from_bytes(bytes(data)) if isinstance(data, (bytes, bytearray, memoryview)) else AprModel.from_path(data)
        md = m.raw_metadata
        if not md.get("classical") or md.get("model_type") not in TYPE_IDS:
            raise ModelError(f"not a classical model file (model_type={md.get('model_type')!r})")
        return cls(md["model_type"], {n: np.array(m.tensor_data(n)).view(np.float32).reshape(t["shape"]) for n, t in m.tensors.items()}, md.get("params") or {}, md.get("feature_names"))

    @property
    def n_features(self) -> int:
        t, p = self.tensors, self.params
        if "coef" in t:
            return int(np.atleast_2d(t["coef"]).shape[-1])
        for k in ("theta", "X", "centers", "components"):
            if k in t:
                return int(t[k].shape[-1])
        return int(p.get("n_features", 0))

    def _trees(self) -> List[Tree]:
        n = int(self.params.get("n_trees", 1))
        return [Tree.from_tensors(self.tensors, f"tree.{i}") for i in range(n)]

    # -- inference ------------------------------------------------------------------------------
    def decision(self, X: np.ndarray) -> np.ndarray:
        """Raw score(s): regression value, margin, per-class probability or log-likelihood."""
        X = np.atleast_2d(np.asarray(X, np.float64))
        if self.n_features and X.shape[1] != self.n_features:
            raise ModelError(f"expected {self.n_features} features, got {X.shape[1]}")
        t, p, mt = self.tensors, self.params, self.model_type
        if mt in ("LinearRegression", "LogisticRegression", "SVM"):
            return X @ np.atleast_2d(t["coef"]).T.astype(np.float64) + np.asarray(t["intercept"], np.float64)
        if mt == "NaiveBayes":
            th, var, prior = t["theta"].astype(np.float64), t["var"].astype(np.float64), t["class_prior"].astype(np.float64)
            ll = -0.5 * (np.log(2 * np.pi * var)[None] + (X[:, None, :] - th[None]) ** 2 / var[None]).sum(-1)
            return ll + np.log(prior)[None]
        if mt == "KNN":
            d = ((X[:, None, :] - t["X"][None].astype(np.float64)) ** 2).sum(-1)
            k = int(p.get("k", 3))
            nn = np.argpartition(d, min(k, d.shape[1] - 1), axis=1)[:, :k]
            labels = t["y"].astype(np.int64)[nn]
            n_cls = int(p.get("n_classes", labels.max() + 1))
            return np.stack([(labels == c).mean(1) for c in range(n_cls)], 1)
        if mt == "KMeans":
            return -((X[:, None, :] - t["centers"][None].astype(np.float64)) ** 2).sum(-1)
        if mt == "PCA":
            return (X - t["mean"].astype(np.float64)) @ t["components"].astype(np.float64).T
        if mt == "DecisionTree":
            return self._trees()[0].predict_value(X)
        if mt == "RandomForest":
            return np.mean([tr.predict_value(X) for tr in self._trees()], axis=0)
        if mt == "GradientBoosting":
            s = float(p.get("init", 0.0)) + float(p.get("learning_rate", 0.1)) * np.sum([tr.predict_value(X) for tr in self._trees()], axis=0)
            return s
        raise ModelError(f"model type '{mt}' has no predictor")

    def predict(self, X) -> np.ndarray:
        z, mt, task = self.decision(X), self.model_type, self.params.get("task", "classification")
        if mt == "LinearRegression" or mt == "PCA":
            return z.squeeze(-1) if mt == "LinearRegression" and z.shape[-1] == 1 else z
        if mt in ("LogisticRegression", "SVM"):
            return (z.squeeze(-1) > 0).astype(np.int64) if z.shape[-1] == 1 else z.argmax(-1)
        if mt in ("NaiveBayes", "KNN", "KMeans"):
            return z.argmax(-1)
        if task == "regression":
            return z
        if mt == "GradientBoosting":
            return (z > 0).astype(np.int64)
        return z.argmax(-1) if z.ndim == 2 else (z > 0.5).astype(np.int64)

    def predict_proba(self, X) -> np.ndarray:
        z, mt = self.decision(X), self.model_type
        if mt == "LogisticRegression":
            if z.shape[-1] == 1:
                p1 = _sigmoid(z.squeeze(-1))
                return np.stack([1 - p1, p1], 1)
            e = np.exp(z - z.max(-1, keepdims=True))
            return e / e.sum(-1, keepdims=True)
        if mt == "NaiveBayes":
            e = np.exp(z - z.max(-1, keepdims=True))
            return e / e.sum(-1, keepdims=True)
        if mt == "GradientBoosting":
            p1 = _sigmoid(z)
            return np.stack([1 - p1, p1], 1)
        if mt in ("KNN", "RandomForest", "DecisionTree") and z.ndim == 2:
            return z / np.maximum(z.sum(-1, keepdims=True), 1e-30)
        raise ModelError(f"model type '{mt}' has no probability output")


# -- explanations ----------------------------------------------------------------------------------------
@dataclass
class ShapExplanation:
    base_value: float
    shap_values: List[float]
    prediction: float
    feature_names: Optional[List[str]] = None

    def top_features(self, n: int = 5) -> List[Tuple[str, float]]:
        names = self.feature_names or [f"feature_{i}" for i in range(len(self.shap_values))]
        return sorted(zip(names, self.shap_values), key=lambda kv: -abs(kv[1]))[:n]

    def verify_consistency(self, tol: float = 1e-3) -> bool:
        """Local accuracy: base + Σφ = prediction."""
        return abs(self.base_value + sum(self.shap_values) - self.prediction) <= tol


def _tree_expected(tr: Tree, node: int = 0) -> float:
    if tr.feature[node] < 0:
        return float(tr.value[node])
    l, r = tr.left[node], tr.right[node]
    return float((tr.cover[l] * _tree_expected(tr, l) + tr.cover[r] * _tree_expected(tr, r)) / tr.cover[node])


def tree_shap(tr: Tree, x: np.ndarray) -> np.ndarray:
    """Path-dependent TreeSHAP (polynomial-time exact Shapley values for one scalar-valued tree)."""
    if tr.cover is None:
        raise ModelError("TreeSHAP needs per-node cover counts")
    phi = np.zeros(x.shape[0])

    def extend(path, pz, po, pi):
        path = [list(p) for p in path] + [[pi, pz, po, 1.0 if not path else 0.0]]
        l = len(path) - 1
        for i in range(l - 1, -1, -1):
            path[i + 1][3] += po * path[i][3] * (i + 1) / (l + 1)
            path[i][3] = pz * path[i][3] * (l - i) / (l + 1)
        return path

    def unwind(path, i):
        l = len(path) - 1
        path = [list(p) for p in path]
        n = path[l][3]
        po, pz = path[i][2], path[i][1]
        for j in range(l - 1, -1, -1):
            if po != 0:
                t = path[j][3]
                path[j][3] = n * (l + 1) / ((j + 1) * po)
                n = t - path[j][3] * pz * (l - j) / (l + 1)
            else:
                path[j][3] = path[j][3] * (l + 1) / (pz * (l - j))
        for j in range(i, l):
            path[j][0], path[j][1], path[j][2] = path[j + 1][0], path[j + 1][1], path[j + 1][2]
        return path[:l]

    def unwound_sum(path, i):
        l = len(path) - 1
        po, pz = path[i][2], path[i][1]
        n, tot = path[l][3], 0.0
        for j in range(l - 1, -1, -1):
            if po != 0:
                t = n * (l + 1) / ((j + 1) * po)
                tot += t
                n = path[j][3] - t * pz * (l - j) / (l + 1)
            else:
                tot += path[j][3] * (l + 1) / (pz * (l - j))
        return tot

    def recurse(node, path, pz, po, pi):
        path = extend(path, pz, po, pi)
        f = tr.feature[node]
        if f < 0:
            for i in range(1, len(path)):
                phi[path[i][0]] += unwound_sum(path, i) * (path[i][2] - path[i][1]) * float(tr.value[node])
            return
        hot, cold = (tr.left[node], tr.right[node]) if x[f] <= tr.threshold[node] else (tr.right[node], tr.left[node])
        iz, io = 1.0, 1.0
        k = next((i for i in range(1, len(path)) if path[i][0] == f), None)
        if k is not None:
            iz, io = path[k][1], path[k][2]
            path = unwind(path, k)
        recurse(hot, path, iz * tr.cover[hot] / tr.cover[node], io, f)
        recurse(cold, path, iz * tr.cover[cold] / tr.cover[node], 0.0, f)

    recurse(0, [], 1.0, 1.0, -1)
    return phi


class ShapExplainer:
    """Linear models: φ_i = w_i (x_i − E[x_i]) against a background mean.  Trees / forests /
    boosting: TreeSHAP per tree, combined with the ensemble's weights."""

    def __init__(self, model: ClassicalModel, background_mean: Optional[np.ndarray] = None):
        self.model = model
        self.bg = None if background_mean is None else np.asarray(background_mean, np.float64)

    def explain(self, x: Sequence[float]) -> ShapExplanation:
        m, x = self.model, np.asarray(x, np.float64)
        mt = m.model_type
        if mt in ("LinearRegression", "LogisticRegression", "SVM"):
            w = np.atleast_2d(m.tensors["coef"]).astype(np.float64)[0]
            b = float(np.atleast_1d(m.tensors["intercept"])[0])
            bg = self.bg if self.bg is not None else np.zeros_like(x)
            return ShapExplanation(float(w @ bg + b), list(w * (x - bg)), float(w @ x + b), m.feature_names)
        if mt in ("DecisionTree", "RandomForest", "GradientBoosting"):
            trees = m._trees()
            if any(t.value.ndim > 1 for t in trees):
                raise ModelError("TreeSHAP is implemented for scalar-valued trees")
            scale = float(m.params.get("learning_rate", 0.1)) if mt == "GradientBoosting" else 1.0 / len(trees)
            phi = scale * np.sum([tree_shap(t, x) for t in trees], axis=0)
            base = scale * sum(_tree_expected(t) for t in trees) + (float(m.params.get("init", 0.0)) if mt == "GradientBoosting" else 0.0)
            return ShapExplanation(base, list(phi), float(np.atleast_1d(m.decision(x[None]))[0]), m.feature_names)
        raise ModelError(f"no explainer for model type '{mt}'")


# -- audit ---------------------------------------------------------------------------------------------------
@dataclass
class LatencyBreakdown:
    preprocessing_ms: float = 0.0
    inference_ms: float = 0.0
    postprocessing_ms: float = 0.0
    explanation_ms: Optional[float] = None

    def total_ms(self) -> float:
        return self.preprocessing_ms + self.inference_ms + self.postprocessing_ms + (self.explanation_ms or 0.0)


@dataclass
class AuditRecord:
    request_id: str
    model_hash: str
    model_type: str
    timestamp: float = field(default_factory=time.time)
    client_hash: Optional[str] = None
    model_version: Optional[str] = None
    input_dims: Optional[List[int]] = None
    input_hash: Optional[str] = None
    prediction: Any = None
    confidence: Optional[float] = None
    latency_ms: Optional[float] = None
    latency_breakdown: Optional[LatencyBreakdown] = None
    warnings: List[str] = field(default_factory=list)
    nan_check_passed: Optional[bool] = None
    confidence_check_passed: Optional[bool] = None
    explanation: Optional[dict] = None

    @classmethod
    def new(cls, model_hash: str, model_type: str) -> "AuditRecord":
        return cls(str(uuid.uuid4()), model_hash, model_type)

    def to_json(self) -> str:
        return json.dumps(asdict(self), default=str)


def hash_input(x: np.ndarray) -> str:
    """Inputs are stored only as a digest (no raw features in the audit trail)."""
    return hashlib.sha256(np.ascontiguousarray(x, np.float32).tobytes()).hexdigest()[:16]


class InMemoryAuditSink:
    def __init__(self, capacity: int = 10000):
        self._r: Dict[str, AuditRecord] = {}
        self.capacity = capacity

    def write(self, rec: AuditRecord) -> None:
        if len(self._r) >= self.capacity:
            self._r.pop(next(iter(self._r)))
        self._r[rec.request_id] = rec

    def get(self, request_id: str) -> Optional[AuditRecord]:
        return self._r.get(request_id)

    def records(self) -> List[AuditRecord]:
        return list(self._r.values())

    def count(self) -> int:
        return len(self._r)


class JsonFileAuditSink:
    """Append-only JSON-lines file."""

    def __init__(self, path: str):
        self.path = path

    def write(self, rec: AuditRecord) -> None:
        with open(self.path, "a") as f:
            f.write(rec.to_json() + "\n")

    def records(self) -> List[dict]:
        try:
            with open(self.path) as f:
                return [json.loads(l) for l in f if l.strip()]
        except FileNotFoundError:
            return []


@dataclass
class ProvenanceChain:
    training_data_hash: Optional[str] = None
    code_sha: Optional[str] = None
    training_env: Dict[str, str] = field(default_factory=dict)
    distillation: List[dict] = field(default_factory=list)
    quantization: Optional[dict] = None
    signatures: List[dict] = field(default_factory=list)

    def add_distillation(self, teacher_hash: str, method: str = "", temperature: float = 1.0) -> None:
        self.distillation.append({"teacher_hash": teacher_hash, "method": method, "temperature": temperature})

    def add_signature(self, signer: str, algorithm: str, signature: str) -> None:
        self.signatures.append({"signer": signer, "algorithm": algorithm, "signature": signature, "timestamp": time.time()})


# -- serving state and Lambda-style handler --------------------------------------------------------------
class ClassicalServeState:
    """What ``/v1/predict``, ``/v1/explain`` and ``/v1/audit/{id}`` run against."""

    def __init__(self, model: ClassicalModel, model_bytes: Optional[bytes] = None, version: str = "1", sink=None, background_mean=None,
                 confidence_threshold: Optional[float] = None):
        self.model, self.version = model, version
        self.model_hash = hashlib.sha256(model_bytes if model_bytes is not None else model.to_apr()).hexdigest()[:16]
        self.sink = sink or InMemoryAuditSink()
        self.explainer = ShapExplainer(model, background_mean)
        self.confidence_threshold = confidence_threshold
        self.requests = 0

    def predict(self, features: Sequence[float], explain: bool = False, client: Optional[str] = None) -> dict:
        t0 = time.perf_counter()
        x = np.asarray(features, np.float64)
        if x.ndim != 1:
            raise ModelError("features must be a flat list")
        t1 = time.perf_counter()
        pred = self.model.predict(x[None])[0]
        conf = None
        try:
            conf = float(self.model.predict_proba(x[None])[0].max())
        except ModelError:
            pass
        t2 = time.perf_counter()
        rec = AuditRecord.new(self.model_hash, self.model.model_type)
        rec.model_version, rec.input_dims, rec.input_hash = self.version, [int(x.shape[0])], hash_input(x)
        rec.client_hash = hashlib.sha256(client.encode()).hexdigest()[:16] if client else None
        rec.prediction = pred.tolist() if isinstance(pred, np.ndarray) else (int(pred) if isinstance(pred, (np.integer, int)) else float(pred))
        rec.confidence = conf
        rec.nan_check_passed = bool(np.isfinite(x).all() and np.isfinite(np.asarray(pred, np.float64)).all())
        rec.confidence_check_passed = None if self.confidence_threshold is None or conf is None else conf >= self.confidence_threshold
        if rec.confidence_check_passed is False:
            rec.warnings.append(f"confidence {conf:.3f} below threshold {self.confidence_threshold}")
        expl_ms = None
        if explain:
            te = time.perf_counter()
            e = self.explainer.explain(x)
            rec.explanation = {"base_value": e.base_value, "shap_values": e.shap_values, "top_features": e.top_features()}
            expl_ms = 1e3 * (time.perf_counter() - te)
        t3 = time.perf_counter()
        rec.latency_breakdown = LatencyBreakdown(1e3 * (t1 - t0), 1e3 * (t2 - t1), 1e3 * (t3 - t2) - (expl_ms or 0.0), expl_ms)
        rec.latency_ms = rec.latency_breakdown.total_ms()
        self.sink.write(rec)
        self.requests += 1
        out = {"request_id": rec.request_id, "model": self.model.model_type, "prediction": rec.prediction, "confidence": conf, "latency_ms": rec.latency_ms}
        if explain:
            out["explanation"] = rec.explanation
        return out


@dataclass
class LambdaMetrics:
    requests_total: int = 0
    requests_success: int = 0
    requests_failed: int = 0
    total_latency_ms: float = 0.0
    cold_starts: int = 0
    batch_requests: int = 0

    def avg_latency_ms(self) -> float:
        return self.total_latency_ms / self.requests_success if self.requests_success else 0.0

    def to_prometheus(self) -> str:
        return "\n".join(f"# TYPE lambda_{k} counter\nlambda_{k} {v}" for k, v in asdict(self).items()) + f"\nlambda_latency_avg_ms {self.avg_latency_ms()}\n"


class LambdaHandler:
    """Single-call deployment shape: model bytes in, ``handle({"features": [...]})`` per invocation;
    the first call is the cold start (the model is parsed lazily and the time recorded)."""

    def __init__(self, model_bytes: bytes):
        if not model_bytes:
            raise ModelError("model bytes are empty")
        if model_bytes[:3] != b"APR":
            raise ModelError("model bytes do not start with the APR magic")
        self.model_bytes = model_bytes
        self.state: Optional[ClassicalServeState] = None
        self.cold_start_ms: Optional[float] = None
        self.metrics = LambdaMetrics()

    @property
    def is_cold_start(self) -> bool:
        return self.state is None

    def _ensure(self) -> ClassicalServeState:
        if self.state is None:
            t = time.perf_counter()
            self.state = ClassicalServeState(ClassicalModel.from_apr(self.model_bytes), self.model_bytes)
            self.cold_start_ms = 1e3 * (time.perf_counter() - t)
            self.metrics.cold_starts += 1
        return self.state

    def handle(self, request: dict) -> dict:
        self.metrics.requests_total += 1
        cold = self.is_cold_start
        t = time.perf_counter()
        try:
            feats = request.get("features")
            if not feats:
                raise ModelError("request has no features")
            r = self._ensure().predict(feats, explain=bool(request.get("explain")))
        except Exception:
            self.metrics.requests_failed += 1
            raise
        ms = 1e3 * (time.perf_counter() - t)
        self.metrics.requests_success += 1
        self.metrics.total_latency_ms += ms
        return {"prediction": r["prediction"], "probabilities": None, "latency_ms": ms, "cold_start": cold, "request_id": r["request_id"],
                **({"explanation": r["explanation"]} if "explanation" in r else {})}

    def handle_batch(self, request: dict) -> dict:
        self.metrics.batch_requests += 1
        t = time.perf_counter()
        out, errors = [], 0
        for inst in request.get("instances", []):
            try:
                out.append(self.handle(inst))
            except Exception as e:
                errors += 1
                out.append({"error": str(e)})
        return {"predictions": out, "success_count": len(out) - errors, "error_count": errors, "total_latency_ms": 1e3 * (time.perf_counter() - t)}
