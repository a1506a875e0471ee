"""APR v2 container: reader (native index parser, optional LZ4 / ZSTD payload), writer, and the
mapping from APR / HuggingFace tensor names and metadata aliases to the engine's GGUF-style names.

Reference parity: ``AprHeader`` / ``TensorEntry`` / ``AprV2Model`` (src/apr/mod.rs:80-403),
metadata aliases (src/apr/metadata.rs:15-90), whole-payload compression
(src/apr/loading_mmap.rs:159-190), HF-style tensor names (src/apr/forward.rs:150-262).
"""
from __future__ import annotations

import ctypes
import ctypes.util
import json
import mmap
import re
import struct
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np

from .._native import cpu_lib
from ..quant import QType, tensor_bytes

HEADER_SIZE, ALIGNMENT = 64, 64
FLAG_LZ4, FLAG_ZSTD, FLAG_ENCRYPTED, FLAG_SIGNED, FLAG_SHARDED, FLAG_QUANTIZED, FLAG_HAS_VOCAB = 1, 2, 4, 8, 0x10, 0x20, 0x200
APR_Q4, APR_Q8 = 128, 129


class AprError(ValueError):
    pass


def _lib(name):
    path = ctypes.util.find_library(name)
    return ctypes.CDLL(path) if path else None


def lz4_decompress_size_prepended(buf: bytes) -> bytes:
    lib = _lib("lz4")
    if lib is None:
        raise AprError("LZ4-compressed .apr file but liblz4 is not available")
    n = struct.unpack_from("<I", buf, 0)[0]
    out = ctypes.create_string_buffer(n)
    got = lib.LZ4_decompress_safe(ctypes.c_char_p(bytes(buf[4:])), out, len(buf) - 4, n)
    if got != n:
        raise AprError("LZ4 decompression failed")
    return out.raw


def lz4_compress_size_prepended(buf: bytes) -> bytes:
    lib = _lib("lz4")
    if lib is None:
        raise AprError("liblz4 is not available")
    bound = lib.LZ4_compressBound(len(buf))
    out = ctypes.create_string_buffer(bound)
    n = lib.LZ4_compress_default(ctypes.c_char_p(buf), out, len(buf), bound)
    return struct.pack("<I", len(buf)) + out.raw[:n]


def zstd_decompress(buf: bytes) -> bytes:
    lib = _lib("zstd")
    if lib is None:
        raise AprError("ZSTD-compressed .apr file but libzstd is not available")
    lib.ZSTD_getFrameContentSize.restype = ctypes.c_ulonglong
    lib.ZSTD_decompress.restype = ctypes.c_size_t
    n = lib.ZSTD_getFrameContentSize(ctypes.c_char_p(bytes(buf)), ctypes.c_size_t(len(buf)))
    if n >= (1 << 62):
        raise AprError("ZSTD frame has no content size")
    out = ctypes.create_string_buffer(n)
    got = lib.ZSTD_decompress(out, ctypes.c_size_t(n), ctypes.c_char_p(bytes(buf)), ctypes.c_size_t(len(buf)))
    if got != n:
        raise AprError("ZSTD decompression failed")
    return out.raw


def zstd_compress(buf: bytes, level: int = 3) -> bytes:
    lib = _lib("zstd")
    if lib is None:
        raise AprError("libzstd is not available")
    lib.ZSTD_compressBound.restype = ctypes.c_size_t
    lib.ZSTD_compress.restype = ctypes.c_size_t
    bound = lib.ZSTD_compressBound(ctypes.c_size_t(len(buf)))
    out = ctypes.create_string_buffer(bound)
    n = lib.ZSTD_compress(out, ctypes.c_size_t(bound), ctypes.c_char_p(buf), ctypes.c_size_t(len(buf)), level)
    return out.raw[:n]


_ALIASES = {"hidden_size": ("hidden_size", "hidden_dim", "d_model", "n_embd"),
            "num_layers": ("num_layers", "n_layers", "num_hidden_layers", "n_layer"),
            "num_heads": ("num_heads", "n_heads", "num_attention_heads", "n_head"),
            "num_kv_heads": ("num_kv_heads", "n_kv_heads", "num_key_value_heads"),
            "vocab_size": ("vocab_size", "n_vocab"),
            "intermediate_size": ("intermediate_size", "ffn_dim", "intermediate_dim", "n_inner"),
            "max_position_embeddings": ("max_position_embeddings", "max_seq_len", "context_length", "n_ctx"),
            "rms_norm_eps": ("rms_norm_eps", "layer_norm_eps", "norm_eps"),
            "rope_theta": ("rope_theta",), "architecture": ("architecture", "model_type")}


def normalise_metadata(meta: dict) -> dict:
    """Collapse the accepted aliases onto HuggingFace-style keys."""
    out = dict(meta)
    for canon, names in _ALIASES.items():
        for n in names:
            if n in meta and meta[n] is not None:
                out[canon] = meta[n]
                break
    return out


class AprModel:
    def __init__(self, data, keepalive=None):
        self._keep = keepalive
        self._np = np.frombuffer(data, dtype=np.uint8)
        lib = cpu_lib()
        lib.rlz_apr_parse.restype = ctypes.c_void_p
        lib.rlz_apr_parse.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
        lib.rlz_apr_free.argtypes = [ctypes.c_void_p]
        rc, err = ctypes.c_int(0), ctypes.create_string_buffer(512)
        p = lib.rlz_apr_parse(self._np.ctypes.data_as(ctypes.c_void_p), self._np.size, ctypes.byref(rc), err, 512)
        if not p:
            raise AprError(err.value.decode("utf-8", "replace"))
        doc = json.loads(ctypes.string_at(p).decode("utf-8", "surrogateescape"))
        lib.rlz_apr_free(p)
        self.header = {k: v for k, v in doc.items() if k != "tensors"}
        self.flags = doc["flags"]
        if self.flags & FLAG_ENCRYPTED:
            raise AprError("encrypted .apr files are not supported")
        mo, ms = doc["metadata_offset"], doc["metadata_size"]
        try:
            self.raw_metadata = json.loads(bytes(self._np[mo: mo + ms]).decode("utf-8")) if ms else {}
        except Exception as e:
            raise AprError(f"invalid .apr metadata JSON: {e}") from e
        self.metadata = normalise_metadata(self.raw_metadata)
        self.tensors: Dict[str, dict] = {t["name"]: t for t in doc["tensors"]}

    @classmethod
    def from_bytes(cls, data: bytes) -> "AprModel":
        if len(data) >= 8 and data[:3] == b"APR":
            flags = struct.unpack_from("<H", data, 6)[0]
            if flags & FLAG_LZ4:
                data = data[:HEADER_SIZE] + lz4_decompress_size_prepended(data[HEADER_SIZE:])
            elif flags & FLAG_ZSTD:
                data = data[:HEADER_SIZE] + zstd_decompress(data[HEADER_SIZE:])
        return cls(bytes(data))

    @classmethod
    def from_path(cls, path) -> "AprModel":
        f = open(path, "rb")
        head = f.read(8)
        flags = struct.unpack_from("<H", head, 6)[0] if len(head) >= 8 and head[:3] == b"APR" else 0
        if flags & (FLAG_LZ4 | FLAG_ZSTD):
            f.seek(0)
            return cls.from_bytes(f.read())
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return cls(mm, keepalive=(f, mm))

    def qtype_of(self, name: str) -> int:
        d = self.tensors[name]["dtype"]
        if d in (APR_Q4, 8):                      # APR-native q4 (and its legacy id) share the Q4_0 block layout
            spec_q4 = tensor_bytes(QType.Q4_0, self.tensors[name]["shape"]) if self.tensors[name]["shape"][-1] % 32 == 0 else -1
            if d == APR_Q4 or self.tensors[name]["size"] == spec_q4:
                return int(QType.Q4_0)
        return int(d)

    def tensor_data(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return self._np[t["offset"]: t["offset"] + t["size"]]

    def vocabulary(self) -> Optional[List[str]]:
        tk = self.raw_metadata.get("tokenizer") or {}
        return self.raw_metadata.get("vocab") or self.raw_metadata.get("vocabulary") or tk.get("vocab") or tk.get("vocabulary")

    def merges(self) -> Optional[List[str]]:
        tk = self.raw_metadata.get("tokenizer") or {}
        return self.raw_metadata.get("merges") or tk.get("merges")


class AprBuilder:
    def __init__(self, metadata: Optional[dict] = None, compression: Optional[str] = None):
        self.metadata = dict(metadata or {})
        self.compression = compression
        self._tensors: List[tuple] = []

    def add_tensor_raw(self, name: str, shape, dtype: int, data) -> "AprBuilder":
        arr = np.ascontiguousarray(np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1))
        self._tensors.append((name, tuple(int(s) for s in shape), int(dtype), arr))
        return self

    def build(self) -> bytes:
        meta = json.dumps(self.metadata).encode()
        flags = 0
        if any(t[2] not in (int(QType.F32), int(QType.F16), int(QType.BF16)) for t in self._tensors):
            flags |= FLAG_QUANTIZED
        if self.metadata.get("vocab") or (self.metadata.get("tokenizer") or {}).get("vocab"):
            flags |= FLAG_HAS_VOCAB
        index, offsets, off = [], [], 0
        for name, shape, dtype, arr in self._tensors:
            offsets.append(off)
            off += (arr.size + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
        for (name, shape, dtype, arr), o in zip(self._tensors, offsets):
            nb = name.encode()
            index.append(struct.pack("<H", len(nb)) + nb + struct.pack("<BB", dtype, len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
                         + struct.pack("<QQ", o, arr.size))
        index_b = b"".join(index)
        meta_off = HEADER_SIZE
        index_off = meta_off + len(meta)
        data_off = (index_off + len(index_b) + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
        body = bytearray(meta + index_b)
        body.extend(b"\0" * (data_off - HEADER_SIZE - len(body)))
        for _, _, _, arr in self._tensors:
            body.extend(arr.tobytes())
            body.extend(b"\0" * ((-arr.size) % ALIGNMENT))
        if self.compression == "lz4":
            flags |= FLAG_LZ4
        elif self.compression == "zstd":
            flags |= FLAG_ZSTD
        head = bytearray(HEADER_SIZE)
        head[0:4] = b"APR2"
        head[4:6] = bytes([2, 0])
        struct.pack_into("<HI", head, 6, flags, len(self._tensors))
        struct.pack_into("<Q", head, 12, meta_off)
        struct.pack_into("<I", head, 20, len(meta))
        struct.pack_into("<Q", head, 24, index_off)
        struct.pack_into("<Q", head, 32, data_off)
        crc = cpu_lib().rlz_crc32
        crc.restype = ctypes.c_uint32
        crc.argtypes = [ctypes.c_char_p, ctypes.c_uint64]
        struct.pack_into("<I", head, 40, crc(bytes(head[:40]), 40))
        payload = bytes(body)
        if self.compression == "lz4":
            payload = lz4_compress_size_prepended(payload)
        elif self.compression == "zstd":
            payload = zstd_compress(payload)
        return bytes(head) + payload

    def write(self, path) -> Path:
        Path(path).write_bytes(self.build())
        return Path(path)


# ------------------------------------------------------------------ tensor-name mapping ----
_HF_LAYER = [("input_layernorm", "attn_norm"), ("post_attention_layernorm", "ffn_norm"), ("self_attn.q_proj", "attn_q"), ("self_attn.k_proj", "attn_k"),
             ("self_attn.v_proj", "attn_v"), ("self_attn.o_proj", "attn_output"), ("self_attn.qkv_proj", "attn_qkv"), ("self_attn.dense", "attn_output"),
             ("self_attn.q_norm", "attn_q_norm"), ("self_attn.k_norm", "attn_k_norm"), ("mlp.gate_proj", "ffn_gate"), ("mlp.up_proj", "ffn_up"),
             ("mlp.down_proj", "ffn_down"), ("mlp.fc1", "ffn_up"), ("mlp.fc2", "ffn_down"), ("ln_1", "attn_norm"), ("ln_2", "ffn_norm"),
             ("attn.c_attn", "attn_qkv"), ("attn.c_proj", "attn_output"), ("mlp.c_fc", "ffn_up"), ("mlp.c_proj", "ffn_down")]
_HF_TOP = {"model.embed_tokens": "token_embd", "embed_tokens": "token_embd", "transformer.wte": "token_embd", "wte": "token_embd",
           "transformer.wpe": "token_pos_embd", "wpe": "token_pos_embd", "model.norm": "output_norm", "norm": "output_norm",
           "model.final_layernorm": "output_norm", "transformer.ln_f": "output_norm", "ln_f": "output_norm", "lm_head": "output"}


def to_gguf_name(name: str) -> Optional[str]:
    """HuggingFace / APR tensor name -> GGUF-style name used by the engine (None if unknown).
    Names that already are GGUF-style pass through."""
    if name.startswith(("blk.", "token_embd", "output", "token_pos_embd")):
        return name
    m = re.match(r"^(?:model\.|transformer\.)?(?:layers|h)\.(\d+)\.(.+)\.(weight|bias)$", name)
    if m:
        for hf, gg in _HF_LAYER:
            if m.group(2) == hf:
                return f"blk.{m.group(1)}.{gg}.{m.group(3)}"
        return None
    base, _, suffix = name.rpartition(".")
    if suffix in ("weight", "bias") and base in _HF_TOP:
        return f"{_HF_TOP[base]}.{suffix}"
    return None
