"""Block quantisation: ggml type ids, layout specs and the native quantise / dequantise /
fused mat-vec entry points (reference parity: src/gguf/types.rs:30-120,
src/quantize/mod.rs:14-150, src/cuda/types.rs:99-230)."""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass

import numpy as np

from .._native import cpu_lib


class QType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ2_XS = 17
    BF16 = 30


@dataclass(frozen=True)
class BlockSpec:
    elems: int
    nbytes: int

    @property
    def bits_per_weight(self) -> float:
        return 8.0 * self.nbytes / self.elems


BLOCK_SPECS = {
    QType.F32: BlockSpec(1, 4), QType.F16: BlockSpec(1, 2), QType.BF16: BlockSpec(1, 2),
    QType.Q4_0: BlockSpec(32, 18), QType.Q4_1: BlockSpec(32, 20), QType.Q5_0: BlockSpec(32, 22),
    QType.Q5_1: BlockSpec(32, 24), QType.Q8_0: BlockSpec(32, 34), QType.Q8_1: BlockSpec(32, 36),
    QType.Q2_K: BlockSpec(256, 84), QType.Q3_K: BlockSpec(256, 110), QType.Q4_K: BlockSpec(256, 144),
    QType.Q5_K: BlockSpec(256, 176), QType.Q6_K: BlockSpec(256, 210),
}

#: types the engine can execute (quantise, dequantise, CPU mat-vec, GPU kernels)
WEIGHT_TYPES = (QType.F32, QType.F16, QType.BF16, QType.Q4_0, QType.Q4_1, QType.Q5_0, QType.Q5_1,
                QType.Q8_0, QType.Q2_K, QType.Q4_K, QType.Q5_K, QType.Q6_K)


def row_bytes(qtype: int, k: int) -> int:
    spec = BLOCK_SPECS[QType(qtype)]
    if k % spec.elems:
        raise ValueError(f"row length {k} is not a multiple of the {QType(qtype).name} block size {spec.elems}")
    return k // spec.elems * spec.nbytes


def tensor_bytes(qtype: int, shape) -> int:
    shape = tuple(int(s) for s in shape)
    rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
    return rows * row_bytes(qtype, shape[-1])


def qtype_from_size(nbytes: int, n: int, k: int):
    """Guess the block type of an ``n x k`` weight from its byte size (reference:
    WeightQuantType::from_size, src/cuda/types.rs:190)."""
    for t in (QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.Q8_0, QType.Q5_0, QType.Q4_0, QType.Q4_1, QType.F32, QType.F16):
        spec = BLOCK_SPECS[t]
        if k % spec.elems == 0 and n * (k // spec.elems) * spec.nbytes == nbytes:
            return t
    return None


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def quantize(x: np.ndarray, qtype: int) -> np.ndarray:
    """Quantise a float matrix ``[..., k]`` row by row; returns a flat ``uint8`` array."""
    qtype = QType(qtype)
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    rows = x.size // k
    out = np.empty(rows * row_bytes(qtype, k), dtype=np.uint8)
    rc = cpu_lib().rlz_quantize(int(qtype), _ptr(x), _ptr(out), rows, k)
    if rc:
        raise ValueError(f"cannot quantise to {qtype.name} (rc={rc})")
    return out


def dequantize(data, qtype: int, shape) -> np.ndarray:
    """Decode block bytes to float32 with the given logical shape."""
    qtype = QType(qtype)
    shape = tuple(int(s) for s in shape)
    n = int(np.prod(shape))
    buf = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
    need = tensor_bytes(qtype, shape)
    if buf.size < need:
        raise ValueError(f"{qtype.name} tensor of shape {shape} needs {need} bytes, got {buf.size}")
    buf = np.ascontiguousarray(buf[:need])
    out = np.empty(n, dtype=np.float32)
    rc = cpu_lib().rlz_dequantize(int(qtype), _ptr(buf), _ptr(out), n)
    if rc:
        raise ValueError(f"cannot dequantise {qtype.name} (rc={rc})")
    return out.reshape(shape)


def matvec(data, qtype: int, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """``y = W x`` on the CPU straight from block bytes (activations quantised to Q8_K / Q8_0)."""
    buf = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    batch = x.size // k
    y = np.empty((batch, n), dtype=np.float32)
    rc = cpu_lib().rlz_matvec(int(qtype), _ptr(buf), _ptr(x), _ptr(y), n, k, batch)
    if rc:
        raise ValueError(f"matvec failed (rc={rc})")
    return y if x.ndim > 1 else y[0]


# --------------------------------------------------------------------------------------
# Independent numpy decoders for the two Q4_K_M block types (used by tests to cross-check
# the C++ decoders, and by readers who want the layout spelled out).
def _scale_min_k4(sc: np.ndarray):
    """sc: [nb, 12] uint8 -> (scales [nb, 8], mins [nb, 8])."""
    s = np.empty(sc.shape[:-1] + (8,), np.uint8)
    m = np.empty_like(s)
    s[..., :4] = sc[..., 0:4] & 63
    m[..., :4] = sc[..., 4:8] & 63
    s[..., 4:] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    m[..., 4:] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    return s, m


def dequantize_q4_k_numpy(data: np.ndarray, n_elems: int) -> np.ndarray:
    b = np.frombuffer(data, np.uint8)[: n_elems // 256 * 144].reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    s, m = _scale_min_k4(b[:, 4:16])
    qs = b[:, 16:].reshape(-1, 4, 32)
    lo, hi = (qs & 0xF).astype(np.float32), (qs >> 4).astype(np.float32)
    q = np.stack([lo, hi], axis=2).reshape(-1, 8, 32)
    y = d[:, :, None] * s.astype(np.float32)[:, :, None] * q - dmin[:, :, None] * m.astype(np.float32)[:, :, None]
    return y.reshape(-1)


def dequantize_q6_k_numpy(data: np.ndarray, n_elems: int) -> np.ndarray:
    b = np.frombuffer(data, np.uint8)[: n_elems // 256 * 210].reshape(-1, 210)
    ql = b[:, :128].reshape(-1, 2, 64)
    qh = b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].copy().view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
    q1 = (ql[:, :, :32] & 0xF) | (((qh >> 0) & 3) << 4)
    q2 = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
    q3 = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
    q4 = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
    q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32) - 32.0   # [nb, 2, 4, 32]
    scale = sc.reshape(-1, 2, 4, 2).repeat(16, axis=3)                 # is = l//16 + 2*group
    y = d[:, :, None, None] * scale * q
    return y.reshape(-1)
