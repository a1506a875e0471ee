"""Speculative decoding: a cheap draft proposes ``k`` tokens, the target checks all of them in one
batched pass and keeps the longest agreeing prefix plus its own next token, so every round emits
between 1 and ``k + 1`` tokens for one read of the target's weights.

* ``SpeculativeDecoder`` is generic over two ``SpecModel``s (draft, target).
* ``EngineSpecModel`` wraps a GPU ``DecodeEngine`` slot (verification = one tensor-core pass,
  rejected tokens rolled back in the paged KV cache).
* ``LayerSkipDraft`` is the self-speculative draft: the same engine and KV cache, every second
  layer skipped.
* ``CpuSpecModel`` wraps the C++ CPU decoder (tests, CPU-only hosts).
* ``rejection_sample`` is the stochastic acceptance rule (accept with min(1, p/q), resample from
  the residual on reject) that preserves the target distribution.

Reference parity: ``SpeculativeDecoder`` / ``SpeculativeConfig`` / ``VerificationResult``
(src/speculative.rs:30-404), ``generate_speculative_cuda`` (layer-skipping draft) and
``generate_speculative_with_draft`` (src/gguf/cuda/speculative.rs:32-494)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence

import numpy as np


class SpecModel(Protocol):
    position: int

    def forward(self, tokens: Sequence[int]) -> List[int]:
        """Append ``tokens`` to the context; return the greedy next token after each of them."""

    def rollback(self, position: int) -> None: ...


@dataclass
class SpeculativeConfig:
    speculation_k: int = 4
    max_tokens: int = 64
    eos_token_id: Optional[int] = None
    adaptive: bool = False            # shrink / grow k with the running acceptance rate
    min_k: int = 1
    max_k: int = 8


@dataclass
class SpeculativeStats:
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_round(self) -> float:
        return self.emitted / self.rounds if self.rounds else 0.0


@dataclass
class VerificationResult:
    accepted: int
    tokens: List[int]                 # accepted drafts + the target's token at the first mismatch (or the bonus token)


def verify_greedy(drafts: Sequence[int], target_next: Sequence[int]) -> VerificationResult:
    """``target_next[i]`` is the target's choice after the context extended by ``drafts[:i]``."""
    a = 0
    while a < len(drafts) and drafts[a] == target_next[a]:
        a += 1
    return VerificationResult(a, list(drafts[:a]) + [int(target_next[a])])


def rejection_sample(draft_tokens: Sequence[int], q: np.ndarray, p: np.ndarray, rng: np.random.Generator) -> VerificationResult:
    """Stochastic verification.  ``q[i]`` / ``p[i]`` are the draft / target distributions at draft
    position ``i``; ``p`` has one more row (the bonus position)."""
    out: List[int] = []
    for i, t in enumerate(draft_tokens):
        if rng.random() < min(1.0, float(p[i, t]) / max(float(q[i, t]), 1e-30)):
            out.append(int(t))
            continue
        resid = np.maximum(p[i] - q[i], 0.0)
        z = resid.sum()
        out.append(int(rng.choice(len(resid), p=resid / z)) if z > 0 else int(np.argmax(p[i])))
        return VerificationResult(i, out)
    out.append(int(rng.choice(p.shape[1], p=p[len(draft_tokens)] / p[len(draft_tokens)].sum())))
    return VerificationResult(len(draft_tokens), out)


class SpeculativeDecoder:
    def __init__(self, target: SpecModel, draft: SpecModel, config: Optional[SpeculativeConfig] = None, shared_cache: bool = False):
        """``shared_cache``: draft and target are views of one KV cache (self-speculative), so the
        draft's appended entries are rolled back before the target re-runs the same positions."""
        self.target, self.draft, self.cfg, self.shared = target, draft, config or SpeculativeConfig(), shared_cache
        self.stats = SpeculativeStats()

    def generate(self, prompt: Sequence[int], on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        cfg = self.cfg
        if not prompt:
            raise ValueError("empty prompt")
        # the target consumes all but the last prompt token; `last` is always "accepted but not yet fed"
        if len(prompt) > 1:
            self.target.forward(prompt[:-1])
            if not self.shared:
                self.draft.forward(prompt[:-1])
        last = int(prompt[-1])
        draft_pending: List[int] = []          # accepted tokens the (separate) draft has not seen yet
        out: List[int] = []
        k = cfg.speculation_k
        while len(out) < cfg.max_tokens:
            k_now = max(1, min(k, cfg.max_tokens - len(out)))
            pos0 = self.target.position
            drafts: List[int] = []
            feed = draft_pending + [last]
            for _ in range(k_now):
                t = self.draft.forward(feed)[-1]
                drafts.append(int(t))
                feed = [t]
            if self.shared:
                self.target.rollback(pos0)
            nxt = self.target.forward([last] + drafts)
            v = verify_greedy(drafts, nxt)
            self.target.rollback(pos0 + 1 + v.accepted)
            if not self.shared:
                # the draft has consumed last, d1 .. d_{k-1}; keep what is still valid
                self.draft.rollback(min(self.draft.position, pos0 + 1 + v.accepted))
                draft_pending = [drafts[-1]] if v.accepted == k_now else []
            self.stats.rounds += 1
            self.stats.drafted += k_now
            self.stats.accepted += v.accepted
            stop = False
            for t in v.tokens:
                out.append(t)
                self.stats.emitted += 1
                if on_token:
                    on_token(t)
                if t == cfg.eos_token_id or len(out) >= cfg.max_tokens:
                    stop = True
                    break
            if stop:
                break
            last = v.tokens[-1]
            if cfg.adaptive:
                r = v.accepted / k_now
                k = min(cfg.max_k, k + 1) if r > 0.8 else max(cfg.min_k, k - 1) if r < 0.4 else k
        return out


# -- adapters --------------------------------------------------------------------------------------
class EngineSpecModel:
    """One slot of a GPU engine as a ``SpecModel`` (greedy)."""

    def __init__(self, engine, slot: int = 0, reserve: Optional[int] = None):
        self.engine, self.slot = engine, slot
        engine.open_slot(slot, reserve or engine.cfg.max_seq_len)
        from .engine import SamplingParams
        engine.set_sampling(slot, SamplingParams(temperature=0.0, top_k=1))

    @property
    def position(self) -> int:
        return self.engine.slots[self.slot].position

    def forward(self, tokens: Sequence[int]) -> List[int]:
        return self.engine.forward_tokens(self.slot, tokens)

    def rollback(self, position: int) -> None:
        self.engine.rollback(self.slot, position)

    def close(self) -> None:
        self.engine.close_slot(self.slot)


class LayerSkipDraft:
    """Self-speculative draft over the target's own slot and KV cache: runs ``layers`` only
    (default: every second layer, always including the last one)."""

    def __init__(self, target: EngineSpecModel, layers: Optional[Sequence[int]] = None):
        self.t = target
        n = target.engine.mcfg.num_layers
        self.layers = tuple(layers) if layers is not None else tuple(sorted(set(range(0, n, 2)) | {n - 1}))

    @property
    def position(self) -> int:
        return self.t.position

    def forward(self, tokens: Sequence[int]) -> List[int]:
        return [self.t.engine.draft_step(self.t.slot, int(t), self.layers) for t in tokens]

    def rollback(self, position: int) -> None:
        self.t.rollback(position)


class CpuSpecModel:
    def __init__(self, cpu_model):
        self.m, self.position = cpu_model, 0

    def forward(self, tokens: Sequence[int]) -> List[int]:
        out = []
        for t in tokens:
            out.append(int(np.argmax(self.m.forward(int(t), self.position))))
            self.position += 1
        return out

    def rollback(self, position: int) -> None:
        self.position = position
