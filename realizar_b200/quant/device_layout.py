"""Device-side weight layouts.

Checkpoints are read in their stored block layout; at upload a tensor may be *re-strided*
(never re-quantised) so that every lane of the decode GEMV can issue aligned 16-byte loads:

* Q4_K / Q5_K: stored blocks unchanged (144 / 176 bytes are multiples of 16).
* Q6_K: each 210-byte block is followed by 14 pad bytes (224-byte stride).
* Q8_0 / Q4_0: planar rows – all fp16 block scales first (padded to 16 bytes), then the quants.
* everything else: stored bytes, rows padded to a multiple of 16 bytes.

The matching constants live in ``csrc/gemv_units.h``.
"""
from __future__ import annotations

import torch

from . import BLOCK_SPECS, QType

Q6K_DEV_STRIDE = 224
FAST_TYPES = (QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.Q8_0, QType.Q4_0)


def _pad16(n: int) -> int:
    return (n + 15) & ~15


def dev_row_bytes(qtype: int, k: int) -> int:
    qtype = QType(qtype)
    if qtype == QType.Q6_K:
        return k // 256 * Q6K_DEV_STRIDE
    if qtype == QType.Q8_0:
        return _pad16(2 * (k // 32)) + k
    if qtype == QType.Q4_0:
        return _pad16(2 * (k // 32)) + k // 2
    spec = BLOCK_SPECS[qtype]
    return _pad16(k // spec.elems * spec.nbytes)


def to_device_layout(data: torch.Tensor, qtype: int, n: int, k: int) -> torch.Tensor:
    """``data``: flat uint8 tensor of ``n`` rows in the stored layout -> ``[n, dev_row_bytes]`` uint8."""
    qtype = QType(qtype)
    spec = BLOCK_SPECS[qtype]
    nb = k // spec.elems
    src = data.reshape(n, nb, spec.nbytes)
    if qtype == QType.Q6_K:
        out = torch.zeros(n, nb, Q6K_DEV_STRIDE, dtype=torch.uint8, device=data.device)
        out[:, :, :210] = src
        return out.reshape(n, nb * Q6K_DEV_STRIDE)
    if qtype in (QType.Q8_0, QType.Q4_0):
        qoff = _pad16(2 * nb)
        qbytes = spec.nbytes - 2
        out = torch.zeros(n, qoff + nb * qbytes, dtype=torch.uint8, device=data.device)
        out[:, : 2 * nb] = src[:, :, :2].reshape(n, 2 * nb)
        out[:, qoff:] = src[:, :, 2:].reshape(n, nb * qbytes)
        return out
    row = nb * spec.nbytes
    if row % 16 == 0:
        return src.reshape(n, row).contiguous()
    out = torch.zeros(n, _pad16(row), dtype=torch.uint8, device=data.device)
    out[:, :row] = src.reshape(n, row)
    return out
