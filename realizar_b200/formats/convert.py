"""Checkpoint converters: GGUF -> APR (f32 or keeping / re-quantising blocks), SafeTensors -> APR /
GGUF, and whole-model re-quantisation (reference parity: ``GgufToAprConverter``,
``GgufToAprQ4KConverter``, SafeTensors -> APR: src/convert/mod.rs:72-434)."""
from __future__ import annotations

from typing import Optional

import numpy as np

from ..models.weights import ModelWeights, QTensor, weights_to_gguf, _fallback_type
from ..quant import QType, quantize
from .apr import AprBuilder


def requantize(w: ModelWeights, qtype: int, keep_f32_1d: bool = True) -> ModelWeights:
    """Return a copy whose 2-D tensors are stored as ``qtype`` (rows that do not fit a 256-wide
    block fall back to the matching 32-wide type)."""
    out = {}
    for name, t in w.tensors.items():
        if len(t.shape) != 2 or (keep_f32_1d and "norm" in name):
            out[name] = t
            continue
        qt = _fallback_type(QType(qtype), t.shape[1])
        out[name] = t if int(qt) == int(t.qtype) else QTensor(int(qt), t.shape, quantize(t.to_f32(), qt))
    return ModelWeights(w.config, out, w.vocabulary, dict(w.metadata), w._keepalive)     # untouched tensors may still view the source mapping


def weights_to_apr(w: ModelWeights, compression: Optional[str] = None, dequantize_to_f32: bool = False, hf_names: bool = False) -> bytes:
    """Serialise as APR v2 (GGUF-style tensor names; metadata in HuggingFace-style keys)."""
    c = w.config
    meta = {"architecture": c.architecture, "hidden_size": c.hidden_dim, "num_layers": c.num_layers, "num_heads": c.num_heads,
            "num_kv_heads": c.num_kv_heads, "head_dim": c.head_dim, "intermediate_size": c.intermediate_dim, "vocab_size": c.vocab_size,
            "max_position_embeddings": c.context_length, "rope_theta": c.rope_theta, "rope_dim": c.rope_dim,
            "rms_norm_eps": c.eps, "bos_token_id": c.bos_token_id, "eos_token_id": c.eos_token_id}
    if w.vocabulary:
        meta["vocab"] = list(w.vocabulary)
    if w.metadata.get("merges"):
        meta["merges"] = w.metadata["merges"]
    b = AprBuilder(meta, compression)
    for name, t in w.tensors.items():
        if dequantize_to_f32:
            a = t.to_f32()
            b.add_tensor_raw(name, a.shape, int(QType.F32), a.view(np.uint8).reshape(-1))
        else:
            b.add_tensor_raw(name, t.shape, t.qtype, t.numpy_bytes())
    return b.build()


def convert(src_path, dst_path, to: str = "apr", qtype: Optional[str] = None, compression: Optional[str] = None) -> dict:
    """File-to-file conversion used by the CLI.  ``to``: "apr" | "gguf"; ``qtype``: e.g. "Q4_K" to re-quantise."""
    from .detect import load_model
    w = load_model(src_path)
    if qtype:
        w = requantize(w, QType[qtype])
    blob = weights_to_apr(w, compression) if to == "apr" else weights_to_gguf(w)
    with open(dst_path, "wb") as f:
        f.write(blob)
    return {"tensors": len(w.tensors), "bytes": len(blob), "quantization": w.quant_summary()}
