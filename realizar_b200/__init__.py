"""realizar_b200 — a Blackwell-native (sm_100a) LLM inference engine.

GGUF / APR v2 / SafeTensors checkpoints, K-quant block layouts consumed as stored,
hand-written CUDA kernels for decode and prefill, tensor-parallel execution over NVLink peer
memory, continuous batching under CUDA graphs and an OpenAI-compatible server.
"""
__version__ = "0.1.0"

from .quant import QType  # noqa: F401
