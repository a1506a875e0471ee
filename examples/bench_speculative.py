"""Speculative decoding on the CPU engine: target and draft are the same tiny model here, so every
draft is accepted and a round emits k + 1 tokens for one verification pass."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
from realizar_b200.models.config import named_config
from realizar_b200.models.cpu_model import CpuModel
from realizar_b200.models.weights import synthetic_weights
from realizar_b200.runtime.speculative import CpuSpecModel, SpeculativeConfig, SpeculativeDecoder

w = synthetic_weights(named_config("tiny-llama"), seed=0, std=0.05)
dec = SpeculativeDecoder(CpuSpecModel(CpuModel(w, 256)), CpuSpecModel(CpuModel(w, 256)), SpeculativeConfig(speculation_k=4, max_tokens=40))
out = dec.generate([1, 2, 3, 4, 5])
print(out)
print(dec.stats, f"acceptance {dec.stats.acceptance_rate:.2f}, {dec.stats.tokens_per_round:.1f} tokens per round")
