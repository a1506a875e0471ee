"""GGUF container: reader over the native mmap parser, and a writer for building models
(synthetic test / benchmark checkpoints and converters).

Reference parity: ``GGUFModel::from_bytes`` / ``MappedGGUFModel::from_path``
(src/gguf/loader_parse.rs:2-300, src/gguf/model.rs:43-215), the in-memory test builder
(src/gguf/test_factory.rs:28-400) and the metadata key set (src/gguf/keys.rs:14-79).
"""
from __future__ import annotations

import ctypes
import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

import numpy as np

from .._native import cpu_lib
from ..quant import QType, dequantize, quantize, tensor_bytes

GGUF_MAGIC = 0x46554747
GGUF_DEFAULT_ALIGNMENT = 32

# metadata value type ids
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i",
               T_F32: "<f", T_BOOL: "<B", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


class GGUFError(ValueError):
    """Raised for malformed or unsupported GGUF input."""


@dataclass
class GGUFTensorInfo:
    name: str
    shape: tuple          # row-major (outermost first): a [n, k] weight has k contiguous
    ne: tuple             # as stored on disk (innermost first)
    qtype: int
    offset: int           # absolute byte offset in the file
    nbytes: int


class GGUFModel:
    """Parsed GGUF file.  Tensor bytes are exposed as zero-copy ``uint8`` views of the mapping."""

    def __init__(self, handle, keepalive=None):
        self._h = handle
        self._keep = keepalive
        lib = cpu_lib()
        n = ctypes.c_uint64()
        p = lib.rlz_gguf_json(handle, ctypes.byref(n))
        raw = ctypes.string_at(p, n.value)
        doc = json.loads(raw.decode("utf-8", "surrogateescape"))
        self.version: int = doc["version"]
        self.alignment: int = doc["alignment"]
        self.data_start: int = doc["data_start"]
        self.metadata: Dict[str, Any] = {}
        self.metadata_types: Dict[str, int] = {}
        for k, v in doc["metadata"].items():
            val = v["v"]
            if v["t"] in (T_F32, T_F64) and isinstance(val, str):
                val = float(val)
            self.metadata[k] = val
            self.metadata_types[k] = v["t"]
        self.tensors: Dict[str, GGUFTensorInfo] = {}
        for t in doc["tensors"]:
            self.tensors[t["name"]] = GGUFTensorInfo(t["name"], tuple(t["shape"]), tuple(t["ne"]), t["qtype"], t["offset"], t["nbytes"])
        size = lib.rlz_gguf_size(handle)
        base = lib.rlz_gguf_base(handle)
        self.size = size
        self._buf = (ctypes.c_uint8 * size).from_address(base) if size else None
        self._np = np.frombuffer(self._buf, dtype=np.uint8) if size else np.zeros(0, np.uint8)

    # -- constructors ------------------------------------------------------------------
    @classmethod
    def from_bytes(cls, data: bytes) -> "GGUFModel":
        arr = np.frombuffer(bytes(data), dtype=np.uint8)
        err = ctypes.create_string_buffer(512)
        h = cpu_lib().rlz_gguf_open_buffer(arr.ctypes.data_as(ctypes.c_void_p), arr.size, err, 512)
        if not h:
            raise GGUFError(err.value.decode("utf-8", "replace"))
        return cls(h, keepalive=arr)

    @classmethod
    def from_path(cls, path) -> "GGUFModel":
        err = ctypes.create_string_buffer(512)
        h = cpu_lib().rlz_gguf_open_file(str(path).encode(), err, 512)
        if not h:
            raise GGUFError(err.value.decode("utf-8", "replace"))
        return cls(h)

    def close(self):
        if self._h:
            self._np = None
            self._buf = None
            cpu_lib().rlz_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- mapping hints (MappedGGUFModel::advise_* / lock_memory) -----------------------------
    def advise(self, mode: str = "normal") -> None:
        cpu_lib().rlz_gguf_advise(self._h, {"normal": 0, "sequential": 1, "random": 2, "willneed": 3}[mode])

    def lock_memory(self) -> bool:
        return cpu_lib().rlz_gguf_lock(self._h) == 0

    # -- access --------------------------------------------------------------------------
    def get(self, key: str, default=None):
        return self.metadata.get(key, default)

    @property
    def architecture(self) -> str:
        return self.metadata.get("general.architecture", "llama")

    def arch_key(self, suffix: str, default=None):
        return self.metadata.get(f"{self.architecture}.{suffix}", default)

    def has_tensor(self, name: str) -> bool:
        return name in self.tensors

    def tensor_data(self, name: str) -> np.ndarray:
        """Raw block bytes of a tensor (zero-copy view)."""
        t = self.tensors[name]
        if t.nbytes == 0 and int(np.prod(t.shape)) != 0:
            raise GGUFError(f"tensor '{name}' has unsupported type id {t.qtype}")
        return self._np[t.offset: t.offset + t.nbytes]

    def tensor_f32(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return dequantize(self.tensor_data(name), t.qtype, t.shape)

    def vocabulary(self) -> Optional[List[str]]:
        return self.metadata.get("tokenizer.ggml.tokens")


# ----------------------------------------------------------------------------------------
class GGUFBuilder:
    """Builds a GGUF v3 byte string: ``add_*`` metadata and tensors, then ``build()``."""

    def __init__(self, architecture: Optional[str] = None, alignment: int = GGUF_DEFAULT_ALIGNMENT, version: int = 3):
        self._kv: List[tuple] = []
        self._tensors: List[tuple] = []
        self.alignment = alignment
        self.version = version
        if architecture:
            self.add_string("general.architecture", architecture)

    # metadata
    def add(self, key: str, vtype: int, value) -> "GGUFBuilder":
        self._kv.append((key, vtype, value))
        return self

    def add_u32(self, key, v): return self.add(key, T_U32, int(v))
    def add_i32(self, key, v): return self.add(key, T_I32, int(v))
    def add_u64(self, key, v): return self.add(key, T_U64, int(v))
    def add_f32(self, key, v): return self.add(key, T_F32, float(v))
    def add_bool(self, key, v): return self.add(key, T_BOOL, bool(v))
    def add_string(self, key, v): return self.add(key, T_STR, str(v))

    def add_array(self, key, elem_type: int, values: Iterable) -> "GGUFBuilder":
        self._kv.append((key, T_ARR, (elem_type, list(values))))
        return self

    def add_string_array(self, key, values): return self.add_array(key, T_STR, values)

    # tensors
    def add_tensor_raw(self, name: str, shape, qtype: int, data) -> "GGUFBuilder":
        data = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1))
        need = tensor_bytes(qtype, shape)
        if data.size != need:
            raise GGUFError(f"tensor '{name}': {QType(qtype).name} {tuple(shape)} needs {need} bytes, got {data.size}")
        self._tensors.append((name, tuple(int(s) for s in shape), int(qtype), data))
        return self

    def add_tensor(self, name: str, array: np.ndarray, qtype: int = QType.F32) -> "GGUFBuilder":
        """Quantise ``array`` (float) to ``qtype`` and add it."""
        array = np.asarray(array, dtype=np.float32)
        return self.add_tensor_raw(name, array.shape, qtype, quantize(array, qtype))

    # serialisation
    @staticmethod
    def _str(s) -> bytes:
        b = s.encode("utf-8", "surrogateescape") if isinstance(s, str) else bytes(s)
        return struct.pack("<Q", len(b)) + b

    def _value(self, vtype: int, value) -> bytes:
        if vtype == T_STR:
            return self._str(value)
        if vtype == T_ARR:
            et, vals = value
            out = [struct.pack("<IQ", et, len(vals))]
            if et == T_STR:
                out.extend(self._str(v) for v in vals)
            else:
                out.append(np.asarray(vals, dtype=np.dtype(_SCALAR_FMT[et])).tobytes())
            return b"".join(out)
        return struct.pack(_SCALAR_FMT[vtype], value)

    def build(self) -> bytes:
        if self.alignment != GGUF_DEFAULT_ALIGNMENT and not any(k == "general.alignment" for k, _, _ in self._kv):
            self.add_u32("general.alignment", self.alignment)
        head = [struct.pack("<IIQQ", GGUF_MAGIC, self.version, len(self._tensors), len(self._kv))]
        for key, vtype, value in self._kv:
            head.append(self._str(key) + struct.pack("<I", vtype) + self._value(vtype, value))
        offset = 0
        infos = []
        for name, shape, qtype, data in self._tensors:
            ne = tuple(reversed(shape))
            infos.append(self._str(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne)
                         + struct.pack("<IQ", qtype, offset))
            offset += (data.size + self.alignment - 1) // self.alignment * self.alignment
        header = b"".join(head) + b"".join(infos)
        pad = (-len(header)) % self.alignment
        chunks = [header, b"\x00" * pad]
        for _, _, _, data in self._tensors:
            chunks.append(data.tobytes())
            chunks.append(b"\x00" * ((-data.size) % self.alignment))
        return b"".join(chunks)

    def write(self, path) -> Path:
        path = Path(path)
        path.write_bytes(self.build())
        return path
