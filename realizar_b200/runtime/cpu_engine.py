"""Slot engine over the C++ CPU decoder, with the same surface as ``DecodeEngine`` (open/close
slot, set_sampling, prefill, feed) so that the continuous-batching loop and the HTTP server run
without a GPU.  Each slot owns one native model handle (weights are referenced, the KV cache is
per handle).  Parity: the reference serves from its CPU ``OwnedQuantizedModel`` when no GPU is
requested (src/cli/mod_server_commands.rs:361-476, src/api/gguf_handlers.rs)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..models.cpu_model import CpuModel
from ..models.weights import ModelWeights
from ..serving.sampling import GenerationConfig, SamplerChain


@dataclass
class CpuEngineConfig:
    max_batch: int = 2
    max_seq_len: int = 1024


class CpuSlotEngine:
    def __init__(self, weights: ModelWeights, config: Optional[CpuEngineConfig] = None):
        self.cfg = config or CpuEngineConfig()
        self.cfg.max_seq_len = min(self.cfg.max_seq_len, weights.config.context_length)
        self.weights = weights
        self.models: List[Optional[CpuModel]] = [None] * self.cfg.max_batch
        self.pos = [0] * self.cfg.max_batch
        self.samplers: Dict[int, Optional[SamplerChain]] = {}
        self.history: Dict[int, List[int]] = {}
        self.num_pages = self.cfg.max_batch * (-(-self.cfg.max_seq_len // 16))

    def open_slot(self, slot: int, reserve_tokens: int) -> int:
        if self.models[slot] is None:
            self.models[slot] = CpuModel(self.weights, self.cfg.max_seq_len)
        self.pos[slot] = 0
        self.history[slot] = []
        return slot

    def close_slot(self, slot: int) -> None:
        self.pos[slot] = 0
        self.history.pop(slot, None)
        self.samplers.pop(slot, None)

    def set_sampling(self, slot: int, sp) -> None:
        greedy = sp.temperature <= 0 or sp.top_k == 1
        self.samplers[slot] = None if greedy else SamplerChain(GenerationConfig(
            max_tokens=sp.max_tokens, temperature=sp.temperature, top_k=sp.top_k, top_p=sp.top_p, min_p=getattr(sp, "min_p", 0.0)))

    def _pick(self, slot: int, logits: np.ndarray) -> int:
        ch = self.samplers.get(slot)
        return int(np.argmax(logits)) if ch is None else int(ch.sample(logits, self.history[slot]))

    def prefill(self, slot: int, tokens: Sequence[int]) -> int:
        m = self.models[slot]
        logits = m.prefill([int(t) for t in tokens], pos0=self.pos[slot])     # chunks of 32 tokens per batched pass
        self.pos[slot] += len(tokens)
        self.history[slot].extend(int(t) for t in tokens)
        return self._pick(slot, logits)

    def feed(self, slot_tokens: Dict[int, int]) -> List[int]:
        out = [0] * self.cfg.max_batch
        slots = sorted(slot_tokens)
        if len(slots) > 1:                                   # lock-step: the weights are read once for all running sequences
            rows = CpuModel.forward_rows([self.models[s] for s in slots], [int(slot_tokens[s]) for s in slots], [self.pos[s] for s in slots])
        else:
            rows = [self.models[s].forward(int(slot_tokens[s]), self.pos[s]) for s in slots]
        for s, logits in zip(slots, rows):
            self.pos[s] += 1
            self.history[s].append(int(slot_tokens[s]))
            out[s] = self._pick(s, logits)
        return out
