"""Format-neutral weight container and the synthetic checkpoint generator.

``ModelWeights`` is what every loader (GGUF, APR, SafeTensors) produces and what every
runtime (CPU engine, fp32 oracle, GPU engine) consumes: a ``ModelConfig`` plus tensors in
GGUF naming, each kept in its stored block layout (reference parity:
``OwnedQuantizedModel`` / ``OwnedQuantizedTensor`` src/gguf/quantized.rs:26-140 and the GGUF
tensor-name table src/gguf/transformer_loader.rs:18-204).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional

import numpy as np
import torch

from ..quant import BLOCK_SPECS, QType, dequantize, quantize, tensor_bytes
from ..quant.torch_quant import quantize_torch
from .config import ModelConfig


@dataclass
class QTensor:
    """A tensor in its stored layout: ``data`` is a flat uint8 array (numpy or torch)."""
    qtype: int
    shape: tuple
    data: object

    @property
    def nbytes(self) -> int:
        return tensor_bytes(self.qtype, self.shape)

    def numpy_bytes(self) -> np.ndarray:
        if isinstance(self.data, torch.Tensor):
            return self.data.detach().cpu().numpy()
        return self.data

    def torch_bytes(self, device=None) -> torch.Tensor:
        if isinstance(self.data, torch.Tensor):
            return self.data if device is None else self.data.to(device)
        t = torch.from_numpy(np.ascontiguousarray(self.data))
        return t if device is None else t.to(device)

    def to_f32(self) -> np.ndarray:
        return dequantize(self.numpy_bytes(), self.qtype, self.shape)


@dataclass
class ModelWeights:
    config: ModelConfig
    tensors: Dict[str, QTensor] = field(default_factory=dict)
    vocabulary: Optional[list] = None
    metadata: dict = field(default_factory=dict)
    _keepalive: object = None

    def __contains__(self, name): return name in self.tensors
    def __getitem__(self, name) -> QTensor: return self.tensors[name]
    def get(self, name) -> Optional[QTensor]: return self.tensors.get(name)

    def output_weight(self) -> QTensor:
        """lm_head weight; falls back to the token embedding when embeddings are tied."""
        return self.tensors.get("output.weight") or self.tensors["token_embd.weight"]

    def total_bytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())

    def quant_summary(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for t in self.tensors.values():
            out[QType(t.qtype).name] = out.get(QType(t.qtype).name, 0) + t.nbytes
        return out

    @classmethod
    def from_gguf(cls, g) -> "ModelWeights":
        cfg = ModelConfig.from_gguf(g)
        tensors = {name: QTensor(info.qtype, info.shape, g.tensor_data(name)) for name, info in g.tensors.items()
                   if info.nbytes or int(np.prod(info.shape)) == 0}
        return cls(cfg, tensors, g.vocabulary(), dict(g.metadata), g)


# ------------------------------------------------------------------ synthetic models ----
def _fallback_type(qtype: QType, k: int) -> QType:
    """K-quants need rows that are multiples of 256; otherwise fall back to 32-wide blocks."""
    if BLOCK_SPECS[qtype].elems == 256 and k % 256:
        return {QType.Q4_K: QType.Q5_0, QType.Q5_K: QType.Q5_1, QType.Q6_K: QType.Q8_0, QType.Q2_K: QType.Q4_0}[qtype]
    return qtype


def _use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def tensor_plan(cfg: ModelConfig, scheme: str = "Q4_K_M"):
    """Yield ``(name, shape, qtype)`` for every tensor of a decoder with this config.

    ``Q4_K_M`` follows the usual mixture: Q4_K for most matrices, Q6_K for ``output.weight``
    and for ``attn_v`` / ``ffn_down`` in about half of the layers, Q5_K for a fused
    ``attn_qkv``; norms and biases stay F32.  Other schemes name a single block type.
    """
    c = cfg.constraints
    base = QType.Q4_K if scheme == "Q4_K_M" else QType[scheme]
    mixed = scheme == "Q4_K_M"
    H, I, V = cfg.hidden_dim, cfg.intermediate_dim, cfg.vocab_size
    qd, kvd = cfg.q_dim, cfg.kv_dim
    ln = c.norm_type == "layernorm"

    def mat(name, n, k, t=None):
        return (name, (n, k), _fallback_type(t or base, k))

    yield mat("token_embd.weight", V, H, QType.Q6_K if (mixed and c.tied_embeddings) else None)
    if c.positional_encoding == "absolute":
        yield ("token_pos_embd.weight", (cfg.context_length, H), QType.F32)
    for i in range(cfg.num_layers):
        p = f"blk.{i}."
        more = mixed and _use_more_bits(i, cfg.num_layers)
        yield (p + "attn_norm.weight", (H,), QType.F32)
        if ln:
            yield (p + "attn_norm.bias", (H,), QType.F32)
        if cfg.fused_qkv:
            yield mat(p + "attn_qkv.weight", qd + 2 * kvd, H, QType.Q5_K if mixed else None)
            if c.has_bias:
                yield (p + "attn_qkv.bias", (qd + 2 * kvd,), QType.F32)
        else:
            yield mat(p + "attn_q.weight", qd, H)
            yield mat(p + "attn_k.weight", kvd, H)
            yield mat(p + "attn_v.weight", kvd, H, QType.Q6_K if more else None)
            if c.has_bias:
                yield (p + "attn_q.bias", (qd,), QType.F32)
                yield (p + "attn_k.bias", (kvd,), QType.F32)
                yield (p + "attn_v.bias", (kvd,), QType.F32)
        if c.has_qk_norm:
            yield (p + "attn_q_norm.weight", (cfg.head_dim,), QType.F32)
            yield (p + "attn_k_norm.weight", (cfg.head_dim,), QType.F32)
        yield mat(p + "attn_output.weight", H, qd)
        if c.has_bias and ln:
            yield (p + "attn_output.bias", (H,), QType.F32)
        if not cfg.parallel_residual:
            yield (p + "ffn_norm.weight", (H,), QType.F32)
            if ln:
                yield (p + "ffn_norm.bias", (H,), QType.F32)
        if cfg.gated_ffn:
            yield mat(p + "ffn_gate.weight", I, H)
        yield mat(p + "ffn_up.weight", I, H)
        yield mat(p + "ffn_down.weight", H, I, QType.Q6_K if more else None)
        if c.has_bias and ln:
            yield (p + "ffn_up.bias", (I,), QType.F32)
            yield (p + "ffn_down.bias", (H,), QType.F32)
    yield ("output_norm.weight", (H,), QType.F32)
    if ln:
        yield ("output_norm.bias", (H,), QType.F32)
    if not c.tied_embeddings:
        yield mat("output.weight", V, H, QType.Q6_K if mixed else None)
        if c.has_bias and ln:
            yield ("output.bias", (V,), QType.F32)


def synthetic_weights(cfg: ModelConfig, scheme: str = "Q4_K_M", seed: int = 0, device="cpu",
                      std: float = 0.02, exact_quantizer: Optional[bool] = None) -> ModelWeights:
    """Random-init N(0, std) weights quantised into ``scheme``.

    On CPU with small models the iterative C++ quantiser is used (``exact_quantizer``);
    otherwise tensors are generated and quantised with torch ops on ``device``.
    Norm weights are 1 + N(0, std), norm biases and linear biases N(0, std).
    """
    device = torch.device(device)
    n_params = sum(int(np.prod(s)) for _, s, _ in tensor_plan(cfg, scheme))
    if exact_quantizer is None:
        exact_quantizer = device.type == "cpu" and n_params < 50_000_000
    gen = torch.Generator(device=device).manual_seed(seed)
    tensors: Dict[str, QTensor] = {}
    for name, shape, qt in tensor_plan(cfg, scheme):
        if len(shape) == 1:
            w = torch.randn(shape, generator=gen, device=device) * std
            if name.endswith("norm.weight"):
                w = w + 1.0
            tensors[name] = QTensor(int(QType.F32), shape, w.float().contiguous().view(torch.uint8).reshape(-1)
                                    if device.type != "cpu" else w.float().numpy().view(np.uint8).reshape(-1))
            continue
        n, k = shape
        if exact_quantizer:
            w = (torch.randn(n, k, generator=gen, device=device) * std).cpu().numpy()
            tensors[name] = QTensor(int(qt), shape, quantize(w, qt))
        else:
            step = max(1, (64 << 20) // k)
            parts = []
            for r in range(0, n, step):
                w = torch.randn(min(step, n - r), k, generator=gen, device=device) * std
                parts.append(quantize_torch(w, qt))
            data = torch.cat(parts) if len(parts) > 1 else parts[0]
            tensors[name] = QTensor(int(qt), shape, data if device.type != "cpu" else data.numpy())
    return ModelWeights(cfg, tensors, None, {"general.architecture": cfg.architecture, "synthetic.scheme": scheme, "synthetic.seed": seed})


def weights_to_gguf(w: ModelWeights, vocabulary: Optional[Iterable[str]] = None) -> bytes:
    """Serialise weights (and their config) as a GGUF byte string."""
    from ..formats.gguf import GGUFBuilder
    cfg = w.config
    a = cfg.architecture
    b = GGUFBuilder(a)
    b.add_string("general.name", f"synthetic-{a}")
    b.add_u32(f"{a}.embedding_length", cfg.hidden_dim).add_u32(f"{a}.block_count", cfg.num_layers)
    b.add_u32(f"{a}.attention.head_count", cfg.num_heads).add_u32(f"{a}.attention.head_count_kv", cfg.num_kv_heads)
    b.add_u32(f"{a}.attention.key_length", cfg.head_dim).add_u32(f"{a}.attention.value_length", cfg.head_dim)
    b.add_u32(f"{a}.feed_forward_length", cfg.intermediate_dim).add_u32(f"{a}.context_length", cfg.context_length)
    b.add_u32(f"{a}.vocab_size", cfg.vocab_size)
    b.add_f32(f"{a}.rope.freq_base", cfg.rope_theta).add_u32(f"{a}.rope.dimension_count", cfg.rope_dim)
    key = "attention.layer_norm_epsilon" if cfg.uses_layernorm else "attention.layer_norm_rms_epsilon"
    b.add_f32(f"{a}.{key}", cfg.eps)
    if cfg.bos_token_id is not None:
        b.add_u32("tokenizer.ggml.bos_token_id", cfg.bos_token_id)
    if cfg.eos_token_id is not None:
        b.add_u32("tokenizer.ggml.eos_token_id", cfg.eos_token_id)
    vocab = list(vocabulary) if vocabulary is not None else w.vocabulary
    if vocab:
        b.add_string("tokenizer.ggml.model", "gpt2")
        b.add_string_array("tokenizer.ggml.tokens", vocab)
    for name, t in w.tensors.items():
        b.add_tensor_raw(name, t.shape, t.qtype, t.numpy_bytes())
    return b.build()
