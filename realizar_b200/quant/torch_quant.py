"""Vectorised block quantisers written with torch ops (run on CPU or GPU).

They emit exactly the ggml byte layouts (see ``csrc/quant_blocks.h``) using a one-shot
min/max fit per sub-block instead of the iterative search of the C++ quantiser, so a
multi-billion-parameter random-init model can be quantised on the device in seconds.
The C++ decoders read their output unchanged (tests cross-check this).
"""
from __future__ import annotations

import torch

from . import QType


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """float tensor [...] -> uint8 [..., 2] holding its fp16 bits (little endian)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _k4_pack_scales(ls: torch.Tensor, lm: torch.Tensor) -> torch.Tensor:
    """6-bit scales / mins [..., 8] (uint8) -> 12 packed bytes."""
    out = torch.empty(*ls.shape[:-1], 12, dtype=torch.uint8, device=ls.device)
    out[..., 0:4] = ls[..., 0:4] | ((ls[..., 4:8] >> 4) << 6)
    out[..., 4:8] = lm[..., 0:4] | ((lm[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (ls[..., 4:8] & 0xF) | ((lm[..., 4:8] & 0xF) << 4)
    return out


def _affine_kquant(x: torch.Tensor, nmax: int):
    """x [rows, nsb, 8, 32] -> (d16, dmin16, ls, lm, q) with q in [0, nmax]."""
    mn = x.amin(dim=-1).clamp(max=0.0)
    mx = x.amax(dim=-1)
    scale = (mx - mn) / nmax
    mins = -mn
    d = scale.amax(dim=-1, keepdim=True) / 63.0
    dmin = mins.amax(dim=-1, keepdim=True) / 63.0
    ls = torch.where(d > 0, torch.round(scale / d.clamp(min=1e-30)), torch.zeros_like(scale)).clamp(0, 63)
    lm = torch.where(dmin > 0, torch.round(mins / dmin.clamp(min=1e-30)), torch.zeros_like(mins)).clamp(0, 63)
    d16 = d.to(torch.float16)
    dmin16 = dmin.to(torch.float16)
    eff_d = (d16.float() * ls).unsqueeze(-1)
    eff_m = (dmin16.float() * lm).unsqueeze(-1)
    q = torch.where(eff_d > 0, torch.round((x + eff_m) / eff_d.clamp(min=1e-30)), torch.zeros_like(x)).clamp(0, nmax)
    return d16.squeeze(-1), dmin16.squeeze(-1), ls.to(torch.uint8), lm.to(torch.uint8), q.to(torch.uint8)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // 256
    x = w.float().reshape(rows, nsb, 8, 32)
    d16, dmin16, ls, lm, q = _affine_kquant(x, 15)
    out = torch.empty(rows, nsb, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16)
    out[..., 2:4] = _f16_bytes(dmin16)
    out[..., 4:16] = _k4_pack_scales(ls, lm)
    qg = q.reshape(rows, nsb, 4, 2, 32)
    out[..., 16:144] = (qg[..., 0, :] | (qg[..., 1, :] << 4)).reshape(rows, nsb, 128)
    return out.reshape(-1)


def quantize_q5_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // 256
    x = w.float().reshape(rows, nsb, 8, 32)
    d16, dmin16, ls, lm, q = _affine_kquant(x, 31)
    out = torch.empty(rows, nsb, 176, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16)
    out[..., 2:4] = _f16_bytes(dmin16)
    out[..., 4:16] = _k4_pack_scales(ls, lm)
    hi = (q >> 4) & 1                                   # [rows, nsb, 8, 32]; sub-block j -> bit j of qh[l]
    shifts = torch.arange(8, device=w.device, dtype=torch.uint8).view(1, 1, 8, 1)
    out[..., 16:48] = (hi << shifts).sum(dim=2).to(torch.uint8)
    lo = (q & 0xF).reshape(rows, nsb, 4, 2, 32)
    out[..., 48:176] = (lo[..., 0, :] | (lo[..., 1, :] << 4)).reshape(rows, nsb, 128)
    return out.reshape(-1)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // 256
    x = w.float().reshape(rows, nsb, 16, 16)
    amax = x.abs().amax(dim=-1)
    s = amax / 31.0
    d = s.amax(dim=-1, keepdim=True) / 127.0
    sc = torch.where(d > 0, torch.round(s / d.clamp(min=1e-30)), torch.zeros_like(s)).clamp(-128, 127)
    d16 = d.to(torch.float16)
    eff = (d16.float() * sc).unsqueeze(-1)
    q = torch.where(eff > 0, torch.round(x / eff.clamp(min=1e-30)), torch.zeros_like(x)).clamp(-32, 31) + 32
    L = q.to(torch.uint8).reshape(rows, nsb, 2, 4, 32)   # [half, group t, l]
    out = torch.empty(rows, nsb, 210, dtype=torch.uint8, device=w.device)
    lo = L & 0xF
    ql = torch.empty(rows, nsb, 2, 64, dtype=torch.uint8, device=w.device)
    ql[..., :32] = lo[..., 0, :] | (lo[..., 2, :] << 4)
    ql[..., 32:] = lo[..., 1, :] | (lo[..., 3, :] << 4)
    hi = L >> 4
    qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
    out[..., 0:128] = ql.reshape(rows, nsb, 128)
    out[..., 128:192] = qh.reshape(rows, nsb, 64)
    out[..., 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = _f16_bytes(d16.squeeze(-1))
    return out.reshape(-1)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    d = x.abs().amax(dim=-1) / 127.0
    d16 = d.to(torch.float16)
    q = torch.where(d16.unsqueeze(-1) > 0, torch.round(x / d16.float().unsqueeze(-1).clamp(min=1e-30)), torch.zeros_like(x)).clamp(-127, 127)
    out = torch.empty(rows, k // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16)
    out[..., 2:34] = q.to(torch.int8).view(torch.uint8)
    return out.reshape(-1)


def _signed_max(x: torch.Tensor) -> torch.Tensor:
    idx = x.abs().argmax(dim=-1, keepdim=True)
    return x.gather(-1, idx).squeeze(-1)


def quantize_q4_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    d = _signed_max(x) / -8.0
    d16 = d.to(torch.float16)
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d)).unsqueeze(-1)
    q = (x * inv + 8.5).floor().clamp(0, 15).to(torch.uint8)
    out = torch.empty(rows, k // 32, 18, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16)
    out[..., 2:18] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(-1)


def quantize_q5_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    d = _signed_max(x) / -16.0
    d16 = d.to(torch.float16)
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d)).unsqueeze(-1)
    q = (x * inv + 16.5).floor().clamp(0, 31).to(torch.int64)
    out = torch.empty(rows, k // 32, 22, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16)
    bits = ((q >> 4) & 1) << torch.arange(32, device=w.device)
    qh = bits.sum(dim=-1)                                  # 32-bit mask
    for b in range(4):
        out[..., 2 + b] = ((qh >> (8 * b)) & 0xFF).to(torch.uint8)
    lo = (q & 0xF).to(torch.uint8)
    out[..., 6:22] = lo[..., :16] | (lo[..., 16:] << 4)
    return out.reshape(-1)


_TORCH_QUANTIZERS = {QType.Q4_K: quantize_q4_k, QType.Q5_K: quantize_q5_k, QType.Q6_K: quantize_q6_k,
                     QType.Q8_0: quantize_q8_0, QType.Q4_0: quantize_q4_0, QType.Q5_0: quantize_q5_0}


def quantize_torch(w: torch.Tensor, qtype: int) -> torch.Tensor:
    """Quantise a 2-D float tensor; returns flat uint8 block bytes on the same device."""
    qtype = QType(qtype)
    if qtype == QType.F32:
        return w.float().contiguous().view(torch.uint8).reshape(-1)
    if qtype == QType.F16:
        return w.to(torch.float16).contiguous().view(torch.uint8).reshape(-1)
    if qtype == QType.BF16:
        return w.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(-1)
    fn = _TORCH_QUANTIZERS.get(qtype)
    if fn is None:
        raise ValueError(f"no torch quantiser for {qtype.name}")
    if w.dim() != 2:
        w = w.reshape(-1, w.shape[-1])
    # bound temporary memory: quantise in row chunks of ~32M elements
    rows, k = w.shape
    step = max(1, (32 << 20) // k)
    if rows <= step:
        return fn(w)
    return torch.cat([fn(w[r: r + step]) for r in range(0, rows, step)])
