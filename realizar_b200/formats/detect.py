"""Model-format detection by magic bytes / extension, and the unified ``load_model`` entry point
that turns a GGUF, APR v2 or SafeTensors checkpoint into ``ModelWeights``.

Reference parity: ``detect_format`` / ``ModelFormat`` (src/format.rs:23-250), ``detect_model``
(src/model_loader.rs:52-367), load-time validation (``validate_model_load``, src/contract_gate.rs:57-399),
QKV concat / name resolution (src/safetensors/mapped_model.rs:27-470, src/tensor_names.rs).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Optional

import numpy as np

from ..models.config import ModelConfig
from ..models.weights import ModelWeights, QTensor
from ..quant import QType, tensor_bytes
from .apr import AprModel, to_gguf_name
from .gguf import GGUFModel
from .safetensors import SafeTensorsFile, SafeTensorsModel

MAX_MODEL_BYTES = 1 << 40


class FormatError(ValueError):
    pass


def detect_format_bytes(head: bytes) -> str:
    if len(head) >= 4 and head[:4] == b"GGUF":
        return "gguf"
    if len(head) >= 4 and head[:3] == b"APR" and head[3] in (0, ord("1"), ord("2")):
        return "apr"
    if len(head) >= 9:
        n = struct.unpack("<Q", head[:8])[0]
        if 0 < n < 100 * 1024 * 1024 and head[8:9] == b"{":
            return "safetensors"
    return "unknown"


def detect_format(path) -> str:
    p = Path(path)
    if p.is_dir():
        if any(p.glob("*.safetensors")):
            return "safetensors"
        raise FormatError(f"{p} is a directory without .safetensors files")
    if not p.exists():
        raise FormatError(f"model file not found: {p}")
    if p.stat().st_size > MAX_MODEL_BYTES:
        raise FormatError("model file is implausibly large")
    with open(p, "rb") as f:
        fmt = detect_format_bytes(f.read(16))
    if fmt == "unknown":
        ext = {".gguf": "gguf", ".apr": "apr", ".safetensors": "safetensors"}.get(p.suffix.lower())
        if ext is None:
            raise FormatError(f"unrecognised model format (magic bytes and extension '{p.suffix}' unknown)")
        raise FormatError(f"file has extension {p.suffix} but its magic bytes do not match the {ext} format")
    return fmt


def validate_weights(w: ModelWeights) -> dict:
    """Load-time contract: every tensor the architecture needs is present with a consistent shape.
    Returns a small proof record; raises ``FormatError`` otherwise."""
    cfg = w.config
    cfg.validate()
    need = ["token_embd.weight"]
    H, qd, kvd, I = cfg.hidden_dim, cfg.q_dim, cfg.kv_dim, cfg.intermediate_dim
    checks = 0
    for l in range(cfg.num_layers):
        p = f"blk.{l}."
        if p + "attn_qkv.weight" in w:
            exp = {p + "attn_qkv.weight": (qd + 2 * kvd, H)}
        else:
            exp = {p + "attn_q.weight": (qd, H), p + "attn_k.weight": (kvd, H), p + "attn_v.weight": (kvd, H)}
        exp[p + "attn_output.weight"] = (H, qd)
        exp[p + "ffn_up.weight"] = (I, H)
        exp[p + "ffn_down.weight"] = (H, I)
        if cfg.gated_ffn:
            exp[p + "ffn_gate.weight"] = (I, H)
        for name, shape in exp.items():
            t = w.get(name)
            if t is None:
                raise FormatError(f"model is missing tensor '{name}' required by architecture '{cfg.architecture}'")
            if tuple(t.shape) != shape:
                raise FormatError(f"tensor '{name}' has shape {tuple(t.shape)}, expected {shape}")
            if len(np.asarray(t.numpy_bytes()).reshape(-1)) < tensor_bytes(t.qtype, t.shape):
                raise FormatError(f"tensor '{name}' is truncated")
            checks += 1
    for name in need:
        if name not in w:
            raise FormatError(f"model is missing tensor '{name}'")
    ow = w.output_weight()
    if tuple(ow.shape) != (cfg.vocab_size, H):
        raise FormatError(f"lm_head has shape {tuple(ow.shape)}, expected {(cfg.vocab_size, H)}")
    return {"architecture": cfg.architecture, "tensors_checked": checks + 2, "total_bytes": w.total_bytes(), "quantization": w.quant_summary()}


def _weights_from_named(cfg_dict: dict, get_names, get_tensor, arch_hint: Optional[str] = None, vocab=None) -> ModelWeights:
    cfg = ModelConfig.from_hf_dict(cfg_dict, arch_hint)
    tensors = {}
    for name in get_names():
        g = to_gguf_name(name)
        if g is None:
            continue
        tensors[g] = get_tensor(name)
    # Conv1D-style checkpoints (GPT-2) store [in, out]; fused c_attn is already Q|K|V along the output
    if cfg.constraints.weight_layout == "conv1d":
        for k, t in list(tensors.items()):
            if k.endswith(".weight") and len(t.shape) == 2 and "norm" not in k and not k.startswith(("token_embd", "token_pos_embd")):
                a = t.to_f32().T.copy()
                tensors[k] = QTensor(int(QType.F32), a.shape, a.view(np.uint8).reshape(-1))
    cfg.fused_qkv = "blk.0.attn_qkv.weight" in tensors
    return ModelWeights(cfg, tensors, vocab, dict(cfg_dict))


def load_model(path, validate: bool = True) -> ModelWeights:
    """Load any supported checkpoint into the engine's format-neutral container."""
    fmt = detect_format(path)
    if fmt == "gguf":
        w = ModelWeights.from_gguf(GGUFModel.from_path(path))
    elif fmt == "apr":
        a = AprModel.from_path(path)
        md = a.metadata
        if "hidden_size" not in md:
            raise FormatError(".apr metadata has no transformer configuration (hidden_size); classical-ML .apr models are served by serving.classical")

        def get(name):
            t = a.tensors[name]
            return QTensor(a.qtype_of(name), tuple(t["shape"]), a.tensor_data(name))
        w = _weights_from_named(md, lambda: list(a.tensors), get, md.get("architecture"), a.vocabulary())
        w._keepalive = a
        w.metadata["merges"] = a.merges()
    else:
        st = SafeTensorsModel(path)
        if not st.config:
            raise FormatError("SafeTensors checkpoint has no config.json next to it")
        dt = {"F32": QType.F32, "F16": QType.F16, "BF16": QType.BF16}

        def get(name):
            info = st.info(name)
            if info["dtype"] not in dt:
                raise FormatError(f"tensor '{name}' has dtype {info['dtype']}; float weights are required")
            return QTensor(int(dt[info["dtype"]]), info["shape"], st.raw(name))
        vocab = None
        if st.tokenizer_json:
            v = (st.tokenizer_json.get("model") or {}).get("vocab")
            if isinstance(v, dict):
                vocab = [t for t, _ in sorted(v.items(), key=lambda kv: kv[1])]
        w = _weights_from_named(st.config, st.names, get, None, vocab)
        w._keepalive = st
        if st.tokenizer_json:
            w.metadata["merges"] = (st.tokenizer_json.get("model") or {}).get("merges")
        w.metadata["tokenizer_config"] = st.tokenizer_config
    if validate:
        validate_weights(w)
    return w
