"""Host-side sampling library: logit processors, truncation samplers and generation helpers.

The GPU kernels cover the serving hot path (penalties, temperature, top-k, top-p, min-p);
this module is the complete reference implementation over numpy logits with the long tail of
strategies: typical-p, tail-free, eta / epsilon cut-offs, XTC, DRY, mirostat v2, dynamic
temperature, classifier-free guidance, logit bias, stop-sequence detection, token healing,
beam bookkeeping and a prompt cache.

Capability parity with the reference's ``generate`` module (``GenerationConfig``, ``sample_*``,
``LogitProcessorChain``, ``SamplerChain``: src/generate/mod.rs:107-400, src/generate/algorithms.rs:23-420,
src/generate/dry_penalty.rs:15-430, src/generate/dynamic_temperature.rs:14-450).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

NEG_INF = -np.inf


@dataclass
class GenerationConfig:
    max_tokens: int = 64
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    typical_p: float = 1.0
    tfs_z: float = 1.0
    eta_cutoff: float = 0.0
    epsilon_cutoff: float = 0.0
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    mirostat: int = 0
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    dynatemp_range: float = 0.0
    dynatemp_exponent: float = 1.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    penalty_window: int = 64
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_sequence_breakers: Sequence[int] = ()
    logit_bias: Dict[int, float] = field(default_factory=dict)
    stop_token_ids: Sequence[int] = ()
    stop_sequences: Sequence[str] = ()
    seed: Optional[int] = None

    @classmethod
    def greedy(cls, max_tokens: int = 64) -> "GenerationConfig":
        return cls(max_tokens=max_tokens, temperature=0.0, top_k=1)


# ------------------------------------------------------------------ basic transforms -------
def softmax(logits: np.ndarray) -> np.ndarray:
    z = logits - np.max(logits)
    e = np.exp(z, where=np.isfinite(z), out=np.zeros_like(z, dtype=np.float64))
    s = e.sum()
    return e / s if s > 0 else np.full_like(e, 1.0 / len(e))


def apply_temperature(logits: np.ndarray, t: float) -> np.ndarray:
    return logits / t if t > 0 and t != 1.0 else logits


def apply_logit_bias(logits: np.ndarray, bias: Dict[int, float]) -> np.ndarray:
    if not bias:
        return logits
    out = logits.copy()
    for tok, b in bias.items():
        if 0 <= tok < len(out):
            out[tok] += b
    return out


def apply_repetition_penalties(logits: np.ndarray, history: Sequence[int], repetition: float = 1.0, presence: float = 0.0,
                               frequency: float = 0.0) -> np.ndarray:
    """Same arithmetic as the GPU penalties kernel: divide positive / multiply negative logits of seen
    tokens by ``repetition``, then subtract ``presence + frequency * count``."""
    if not len(history) or (repetition == 1.0 and presence == 0.0 and frequency == 0.0):
        return logits
    out = logits.copy()
    toks, counts = np.unique(np.asarray([t for t in history if 0 <= t < len(logits)], dtype=np.int64), return_counts=True)
    if repetition != 1.0:
        v = out[toks]
        out[toks] = np.where(v > 0, v / repetition, v * repetition)
    out[toks] -= presence + frequency * counts
    return out


def top_k_filter(logits: np.ndarray, k: int) -> np.ndarray:
    if k <= 0 or k >= len(logits):
        return logits
    kth = np.partition(logits, -k)[-k]
    return np.where(logits >= kth, logits, NEG_INF)


def top_p_filter(logits: np.ndarray, p: float) -> np.ndarray:
    if p >= 1.0:
        return logits
    order = np.argsort(-logits, kind="stable")
    probs = softmax(logits)[order]
    keep = np.cumsum(probs) - probs < p               # keep tokens until the mass before them reaches p
    keep[0] = True
    out = np.full_like(logits, NEG_INF)
    out[order[keep]] = logits[order[keep]]
    return out


def min_p_filter(logits: np.ndarray, min_p: float) -> np.ndarray:
    if min_p <= 0:
        return logits
    probs = softmax(logits)
    return np.where(probs >= min_p * probs.max(), logits, NEG_INF)


def typical_filter(logits: np.ndarray, mass: float) -> np.ndarray:
    """Locally typical sampling: keep tokens whose surprise is closest to the entropy."""
    if mass >= 1.0:
        return logits
    probs = softmax(logits)
    logp = np.log(np.maximum(probs, 1e-30))
    ent = -(probs * logp).sum()
    dev = np.abs(-logp - ent)
    order = np.argsort(dev, kind="stable")
    keep = np.cumsum(probs[order]) - probs[order] < mass
    keep[0] = True
    out = np.full_like(logits, NEG_INF)
    out[order[keep]] = logits[order[keep]]
    return out


def tfs_filter(logits: np.ndarray, z: float) -> np.ndarray:
    """Tail-free sampling: cut where the normalised second derivative of the sorted probabilities accumulates z."""
    if z >= 1.0 or len(logits) < 3:
        return logits
    order = np.argsort(-logits, kind="stable")
    probs = softmax(logits)[order]
    d2 = np.abs(np.diff(np.diff(probs)))
    if d2.sum() <= 0:
        return logits
    cdf = np.cumsum(d2 / d2.sum())
    last = int(np.searchsorted(cdf, z)) + 1
    out = np.full_like(logits, NEG_INF)
    out[order[: max(1, last)]] = logits[order[: max(1, last)]]
    return out


def eta_filter(logits: np.ndarray, eta_cutoff: float = 0.0, epsilon_cutoff: float = 0.0) -> np.ndarray:
    """Eta sampling: threshold = min(eps, sqrt(eps) * exp(-entropy)); epsilon sampling: fixed threshold."""
    if eta_cutoff <= 0 and epsilon_cutoff <= 0:
        return logits
    probs = softmax(logits)
    thr = epsilon_cutoff
    if eta_cutoff > 0:
        ent = -(probs * np.log(np.maximum(probs, 1e-30))).sum()
        thr = max(thr, min(eta_cutoff, math.sqrt(eta_cutoff) * math.exp(-ent)))
    keep = probs >= thr
    keep[np.argmax(probs)] = True
    return np.where(keep, logits, NEG_INF)


def xtc_filter(logits: np.ndarray, probability: float, threshold: float, rng: np.random.Generator) -> np.ndarray:
    """Exclude-top-choices: with the given probability remove every token above the threshold except the least likely of them."""
    if probability <= 0 or rng.random() >= probability:
        return logits
    probs = softmax(logits)
    above = np.flatnonzero(probs >= threshold)
    if len(above) < 2:
        return logits
    keep_one = above[np.argmin(probs[above])]
    out = logits.copy()
    out[above] = NEG_INF
    out[keep_one] = logits[keep_one]
    return out


def dynamic_temperature(logits: np.ndarray, base: float, rng_range: float, exponent: float = 1.0) -> float:
    """Entropy-scaled temperature in [base - range, base + range]."""
    if rng_range <= 0:
        return base
    probs = softmax(logits)
    finite = np.isfinite(logits).sum()
    if finite <= 1:
        return base
    ent = -(probs * np.log(np.maximum(probs, 1e-30))).sum()
    norm = ent / math.log(finite)
    lo, hi = max(0.0, base - rng_range), base + rng_range
    return lo + (hi - lo) * (norm ** exponent)


def dry_penalty(logits: np.ndarray, history: Sequence[int], multiplier: float, base: float = 1.75, allowed_length: int = 2,
                breakers: Sequence[int] = ()) -> np.ndarray:
    """DRY ("don't repeat yourself"): penalise tokens that would extend a repeated n-gram; the penalty
    grows as multiplier * base^(match_length - allowed_length)."""
    if multiplier <= 0 or len(history) < 2:
        return logits
    h = list(history)
    brk = set(breakers)
    out = logits.copy()
    n = len(h)
    longest: Dict[int, int] = {}
    for i in range(n - 1):                              # position whose successor could be repeated
        if h[i] != h[-1] or h[i] in brk:
            continue
        L = 1
        while i - L >= 0 and L < n - 1 - i + L and h[i - L] == h[n - 1 - L] and h[i - L] not in brk:
            L += 1
            if L > 50:
                break
        nxt = h[i + 1]
        longest[nxt] = max(longest.get(nxt, 0), L)
    for tok, L in longest.items():
        if L >= allowed_length and 0 <= tok < len(out):
            out[tok] -= multiplier * (base ** (L - allowed_length))
    return out


def cfg_combine(cond: np.ndarray, uncond: np.ndarray, scale: float) -> np.ndarray:
    """Classifier-free guidance on log-probabilities."""
    lc = cond - np.logaddexp.reduce(cond)
    lu = uncond - np.logaddexp.reduce(uncond)
    return lu + scale * (lc - lu)


class Mirostat:
    """Mirostat v2: keep the observed surprise near tau by adapting the truncation threshold mu."""

    def __init__(self, tau: float = 5.0, eta: float = 0.1):
        self.tau, self.eta, self.mu = tau, eta, 2.0 * tau

    def sample(self, logits: np.ndarray, rng: np.random.Generator) -> int:
        probs = softmax(logits)
        surprise = -np.log2(np.maximum(probs, 1e-30))
        keep = surprise <= self.mu
        if not keep.any():
            keep[np.argmax(probs)] = True
        p = np.where(keep, probs, 0.0)
        p /= p.sum()
        tok = int(rng.choice(len(p), p=p))
        self.mu -= self.eta * (float(-np.log2(max(p[tok], 1e-30))) - self.tau)
        return tok


# ------------------------------------------------------------------ chains -----------------
class LogitProcessorChain:
    """Ordered list of ``f(logits, history) -> logits`` processors."""

    def __init__(self, processors: Optional[List[Callable]] = None):
        self.processors = list(processors or [])

    def add(self, fn: Callable) -> "LogitProcessorChain":
        self.processors.append(fn)
        return self

    def __call__(self, logits: np.ndarray, history: Sequence[int] = ()) -> np.ndarray:
        for fn in self.processors:
            logits = fn(logits, history)
        return logits


def sample_greedy(logits: np.ndarray) -> int:
    return int(np.argmax(logits))


def sample_from(logits: np.ndarray, rng: np.random.Generator) -> int:
    p = softmax(logits)
    return int(rng.choice(len(p), p=p))


class SamplerChain:
    """The full pipeline for one request: penalties -> bias -> DRY -> temperature (static or dynamic) ->
    top-k -> tail-free -> typical -> top-p -> min-p -> eta/epsilon -> XTC -> draw (or mirostat)."""

    def __init__(self, cfg: GenerationConfig):
        self.cfg = cfg
        self.rng = np.random.default_rng(cfg.seed)
        self.mirostat = Mirostat(cfg.mirostat_tau, cfg.mirostat_eta) if cfg.mirostat else None

    def process(self, logits: np.ndarray, history: Sequence[int] = ()) -> np.ndarray:
        c = self.cfg
        x = np.asarray(logits, dtype=np.float64)
        window = list(history)[-c.penalty_window:] if c.penalty_window > 0 else list(history)
        x = apply_repetition_penalties(x, window, c.repetition_penalty, c.presence_penalty, c.frequency_penalty)
        x = apply_logit_bias(x, c.logit_bias)
        x = dry_penalty(x, history, c.dry_multiplier, c.dry_base, c.dry_allowed_length, c.dry_sequence_breakers)
        if c.temperature <= 0:
            return x
        t = dynamic_temperature(x, c.temperature, c.dynatemp_range, c.dynatemp_exponent)
        x = apply_temperature(x, t)
        x = top_k_filter(x, c.top_k)
        x = tfs_filter(x, c.tfs_z)
        x = typical_filter(x, c.typical_p)
        x = top_p_filter(x, c.top_p)
        x = min_p_filter(x, c.min_p)
        x = eta_filter(x, c.eta_cutoff, c.epsilon_cutoff)
        x = xtc_filter(x, c.xtc_probability, c.xtc_threshold, self.rng)
        return x

    def sample(self, logits: np.ndarray, history: Sequence[int] = ()) -> int:
        x = self.process(logits, history)
        if self.cfg.temperature <= 0 or self.cfg.top_k == 1:
            return sample_greedy(x)
        if self.mirostat is not None:
            return self.mirostat.sample(x, self.rng)
        return sample_from(x, self.rng)


# ------------------------------------------------------------------ generation helpers -----
class StopSequenceDetector:
    """Detects stop strings across token boundaries; ``push`` returns (text safe to emit, stopped)."""

    def __init__(self, stops: Sequence[str]):
        self.stops = [s for s in stops if s]
        self.held = ""
        self.max_len = max((len(s) for s in self.stops), default=0)

    def push(self, text: str) -> Tuple[str, bool]:
        if not self.stops:
            return text, False
        self.held += text
        for s in self.stops:
            i = self.held.find(s)
            if i >= 0:
                out, self.held = self.held[:i], ""
                return out, True
        keep = 0                                            # longest suffix that is a prefix of some stop
        for s in self.stops:
            for L in range(min(len(s) - 1, len(self.held)), 0, -1):
                if self.held.endswith(s[:L]):
                    keep = max(keep, L)
                    break
        out, self.held = self.held[: len(self.held) - keep], self.held[len(self.held) - keep:]
        return out, False

    def flush(self) -> str:
        out, self.held = self.held, ""
        return out


def token_healing_candidates(vocab: Sequence[str], prompt_tail: str) -> List[int]:
    """Token healing: ids of tokens that start with the trailing fragment of the prompt, so the first
    generated token may re-complete a token boundary the prompt cut through."""
    return [i for i, t in enumerate(vocab) if t.startswith(prompt_tail) and len(t) > len(prompt_tail)] if prompt_tail else []


@dataclass(order=True)
class BeamHypothesis:
    score: float
    tokens: List[int] = field(compare=False, default_factory=list)
    finished: bool = field(compare=False, default=False)


class BeamSearch:
    """Book-keeping for beam search: expand every live hypothesis with its best continuations and keep
    the ``width`` best by length-normalised log-probability."""

    def __init__(self, width: int, length_penalty: float = 1.0, eos_token_id: Optional[int] = None):
        self.width, self.length_penalty, self.eos = width, length_penalty, eos_token_id
        self.beams: List[BeamHypothesis] = [BeamHypothesis(0.0, [])]

    def _norm(self, h: BeamHypothesis) -> float:
        return h.score / (max(1, len(h.tokens)) ** self.length_penalty)

    def step(self, logprobs_per_beam: Sequence[np.ndarray]) -> List[BeamHypothesis]:
        cand: List[BeamHypothesis] = []
        for h, lp in zip(self.beams, logprobs_per_beam):
            if h.finished:
                cand.append(h)
                continue
            top = np.argsort(-lp)[: self.width]
            for t in top:
                cand.append(BeamHypothesis(h.score + float(lp[t]), h.tokens + [int(t)], self.eos is not None and int(t) == self.eos))
        cand.sort(key=self._norm, reverse=True)
        self.beams = cand[: self.width]
        return self.beams

    @property
    def done(self) -> bool:
        return all(h.finished for h in self.beams)

    def best(self) -> BeamHypothesis:
        return max(self.beams, key=self._norm)


class PromptCache:
    """LRU cache keyed by the token tuple of a prompt (e.g. cached first-token logits or KV handles)."""

    def __init__(self, capacity: int = 64):
        self.capacity, self._d, self.hits, self.misses = capacity, OrderedDict(), 0, 0

    def get(self, tokens: Sequence[int]):
        k = tuple(tokens)
        if k in self._d:
            self._d.move_to_end(k)
            self.hits += 1
            return self._d[k]
        self.misses += 1
        return None

    def put(self, tokens: Sequence[int], value) -> None:
        k = tuple(tokens)
        self._d[k] = value
        self._d.move_to_end(k)
        while len(self._d) > self.capacity:
            self._d.popitem(last=False)

    def longest_prefix(self, tokens: Sequence[int]):
        best = None
        for k in self._d:
            if len(k) <= len(tokens) and tuple(tokens[: len(k)]) == k and (best is None or len(k) > len(best)):
                best = k
        return (best, self._d[best]) if best is not None else (None, None)
