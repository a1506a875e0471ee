"""SafeTensors reader / writer without third-party dependencies: 8-byte little-endian header
length, JSON header ``{name: {dtype, shape, data_offsets}}``, raw tensor bytes; mmap access,
sharded checkpoints through ``model.safetensors.index.json`` and the sibling ``config.json`` /
``tokenizer.json`` (reference parity: src/safetensors/mod.rs:51-133,
src/safetensors/mapped_model.rs:27-470, src/safetensors/shard.rs)."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np

DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "I32": (np.int32, 4), "I64": (np.int64, 8),
          "U8": (np.uint8, 1), "I8": (np.int8, 1), "BOOL": (np.bool_, 1), "F64": (np.float64, 8), "I16": (np.int16, 2)}
MAX_HEADER = 100 * 1024 * 1024


class SafeTensorsError(ValueError):
    pass


class SafeTensorsFile:
    def __init__(self, buf, keepalive=None):
        self._keep = keepalive
        self._np = np.frombuffer(buf, dtype=np.uint8)
        if self._np.size < 8:
            raise SafeTensorsError("file too small for a SafeTensors header")
        n = struct.unpack("<Q", bytes(self._np[:8]))[0]
        if n > MAX_HEADER or 8 + n > self._np.size:
            raise SafeTensorsError(f"header length {n} exceeds file size or the 100 MB limit")
        try:
            hdr = json.loads(bytes(self._np[8: 8 + n]).decode("utf-8"))
        except Exception as e:
            raise SafeTensorsError(f"invalid header JSON: {e}") from e
        if not isinstance(hdr, dict):
            raise SafeTensorsError("header is not a JSON object")
        self.metadata = hdr.pop("__metadata__", {}) or {}
        self.data_start = 8 + n
        self.tensors: Dict[str, dict] = {}
        for name, t in hdr.items():
            try:
                dtype, shape, (a, b) = t["dtype"], [int(s) for s in t["shape"]], t["data_offsets"]
            except Exception as e:
                raise SafeTensorsError(f"tensor '{name}': malformed entry") from e
            if dtype not in DTYPES:
                raise SafeTensorsError(f"tensor '{name}': unsupported dtype {dtype}")
            want = int(np.prod(shape)) * DTYPES[dtype][1] if shape else DTYPES[dtype][1]
            if a > b or b - a != want or self.data_start + b > self._np.size:
                raise SafeTensorsError(f"tensor '{name}': data_offsets {a}:{b} do not match shape {shape} / file size")
            self.tensors[name] = {"dtype": dtype, "shape": tuple(shape), "start": self.data_start + a, "end": self.data_start + b}

    @classmethod
    def from_bytes(cls, data: bytes) -> "SafeTensorsFile":
        return cls(bytes(data))

    @classmethod
    def from_path(cls, path) -> "SafeTensorsFile":
        f = open(path, "rb")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return cls(mm, keepalive=(f, mm))

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return self._np[t["start"]: t["end"]]

    def numpy(self, name: str) -> np.ndarray:
        """Tensor as a numpy array (BF16 is returned as float32)."""
        t = self.tensors[name]
        raw = self.raw(name)
        if t["dtype"] == "BF16":
            return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(t["shape"])
        return raw.view(DTYPES[t["dtype"]][0]).reshape(t["shape"])


def write_safetensors(tensors: Dict[str, np.ndarray], path=None, metadata: Optional[dict] = None, bf16: Optional[set] = None) -> bytes:
    """Serialise arrays (names in ``bf16`` are stored as BF16).  Returns the bytes; writes them if ``path`` is given."""
    rev = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.int32): "I32", np.dtype(np.int64): "I64",
           np.dtype(np.uint8): "U8", np.dtype(np.int8): "I8", np.dtype(np.bool_): "BOOL", np.dtype(np.float64): "F64"}
    hdr, chunks, off = {}, [], 0
    if metadata:
        hdr["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if bf16 and name in bf16:
            u = a.astype(np.float32).view(np.uint32)
            data = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)).tobytes()
            dt = "BF16"
        else:
            data, dt = a.tobytes(), rev[a.dtype]
        hdr[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(data)]}
        chunks.append(data)
        off += len(data)
    hb = json.dumps(hdr, separators=(",", ":")).encode()
    hb += b" " * ((-len(hb)) % 8)
    blob = struct.pack("<Q", len(hb)) + hb + b"".join(chunks)
    if path is not None:
        Path(path).write_bytes(blob)
    return blob


class SafeTensorsModel:
    """A checkpoint directory or file: one or many shards, ``config.json`` and tokenizer files."""

    def __init__(self, path):
        p = Path(path)
        self.dir = p if p.is_dir() else p.parent
        self.files: List[SafeTensorsFile] = []
        self.where: Dict[str, SafeTensorsFile] = {}
        index = self.dir / "model.safetensors.index.json"
        if p.is_file() and p.suffix == ".safetensors":
            shard_names = [p.name]
        elif index.exists():
            wm = json.loads(index.read_text()).get("weight_map", {})
            shard_names = sorted(set(wm.values()))
        else:
            shard_names = sorted(f.name for f in self.dir.glob("*.safetensors"))
        if not shard_names:
            raise SafeTensorsError(f"no .safetensors files in {self.dir}")
        for s in shard_names:
            f = SafeTensorsFile.from_path(self.dir / s)
            self.files.append(f)
            for name in f.tensors:
                self.where[name] = f
        cfg = self.dir / "config.json"
        self.config: dict = json.loads(cfg.read_text()) if cfg.exists() else {}
        tk = self.dir / "tokenizer.json"
        self.tokenizer_json: Optional[dict] = json.loads(tk.read_text()) if tk.exists() else None
        tc = self.dir / "tokenizer_config.json"
        self.tokenizer_config: Optional[dict] = json.loads(tc.read_text()) if tc.exists() else None

    def names(self) -> List[str]:
        return list(self.where)

    def info(self, name: str) -> dict:
        return self.where[name].tensors[name]

    def numpy(self, name: str) -> np.ndarray:
        return self.where[name].numpy(name)

    def raw(self, name: str) -> np.ndarray:
        return self.where[name].raw(name)
