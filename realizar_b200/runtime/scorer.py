"""Scoring front end of a serving engine: log-probabilities, perplexity and embeddings of given text.

``EngineScorer`` runs ``DecodeEngine.score_tokens`` (tensor-core pass over all rows, head GEMM, log-softmax / gather kernel) on
the engine thread of a ``ServingEngine``, between two scheduling iterations, so scoring requests and streaming generations
share one engine.  The HTTP layer uses it behind ``/v1/logprobs``, ``/v1/perplexity`` and ``/v1/embeddings``.

Reference parity: ``generate_gpu_resident_logprobs`` / ``perplexity_gpu_resident`` / ``perplexity_gpu_batched``
(src/gguf/cuda/generate_2.rs:590-780) and the handlers in src/api/gpu_completions_handler.rs:411-486.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


class EngineScorer:
    def __init__(self, serving, timeout: float = 120.0):
        self.serving, self.timeout = serving, timeout

    def score(self, ids: Sequence[int], want_embedding: bool = False, top_k: int = 0) -> dict:
        ids = [int(t) for t in ids]
        return self.serving.call_on_engine(lambda eng: eng.score_tokens(ids, want_embedding=want_embedding, top_k=top_k), self.timeout)

    def logprobs(self, ids: Sequence[int]) -> List[float]:
        """``log p(ids[i+1] | ids[:i+1])`` for i = 0 .. n-2."""
        return self.score(ids)["logprobs"]

    def embed(self, ids: Sequence[int]) -> List[float]:
        """Mean of the final-norm hidden states over the tokens."""
        return self.score(ids, want_embedding=True)["embedding"]


def scorer_for(serving) -> Optional[EngineScorer]:
    """A scorer when the serving engine's model can run the token-batch path, else None (the endpoints then answer 501)."""
    eng = getattr(serving, "engine", None)
    inner = getattr(eng, "engine", eng)                       # tensor-parallel leader proxies wrap the engine
    if eng is None or not hasattr(eng, "score_tokens") or not getattr(inner, "gemm_ok", False):
        return None
    return EngineScorer(serving)
