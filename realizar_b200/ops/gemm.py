"""Tensor-core dequant-GEMM (tcgen05 / TMEM) over block-quantised weights: prefill and large
decode batches.  ``Y[m, n] = act(X[m, k] W[n, k]^T + bias) + residual`` with X in bf16."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import DeviceWeight, check, lib, ptr, stream_ptr, ACT_NONE
from . import _signatures as S
from ..quant import QType

GM_OUT_BF16, GM_RES_MUL = 1, 2
GEMM_TYPES = (int(QType.Q4_K), int(QType.Q5_K), int(QType.Q6_K), int(QType.BF16), int(QType.F16),
              int(QType.Q4_0), int(QType.Q4_1), int(QType.Q5_0), int(QType.Q5_1), int(QType.Q8_0))     # 32-weight blocks: register-path producers


def gemm_eligible(w: DeviceWeight) -> bool:
    if w.qtype not in GEMM_TYPES:
        return False
    return w.k % 256 == 0 if w.qtype in GEMM_TYPES[:3] else w.k % 64 == 0


def token_tile(m: int) -> int:
    """Tokens per CTA (the MMA N dimension) that the kernel picks for ``m`` tokens."""
    return 32 if m <= 32 else 64 if m <= 64 else 128 if m <= 128 else 256


def choose_splitk(n: int, k: int, m: int, sm_count: int = 148) -> int:
    """Split K across CTAs when the (n, m) tile grid alone would leave most SMs idle; every split
    keeps at least eight 64-column steps so that the pipeline fill is amortised."""
    mt = token_tile(m)
    tiles = -(-n // 128) * -(-m // mt)
    slots = sm_count * (2 if mt <= 64 else 1)
    if tiles >= slots:
        return 1
    return max(1, min(k // 512, slots // tiles, 16))


def build_gemm_params(w: DeviceWeight, x: torch.Tensor, y: torch.Tensor, m: int, bias=None, residual=None, act=ACT_NONE,
                      splitk: int = 1, ldx: Optional[int] = None, ldy: Optional[int] = None, ld_res: Optional[int] = None,
                      wide: int = 0, res_mul: bool = False) -> S.GemmParams:
    """``y`` may be bf16 (the epilogue then writes the operand of the next GEMM directly; not with split-K).
    ``res_mul``: the ``residual`` operand multiplies the activated result instead of being added (gated MLP)."""
    if x.dtype != torch.bfloat16 or y.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("gemm expects bf16 activations and an fp32 or bf16 output")
    if (y.dtype == torch.bfloat16 or res_mul) and splitk > 1:
        raise ValueError("bf16 output and the multiplying operand need an unsplit K")
    p = S.GemmParams()
    p.W, p.w_stride, p.qtype, p.n, p.k, p.m = w.data.data_ptr(), w.stride, w.qtype, w.n, w.k, m
    p.X, p.ldx = x.data_ptr(), ldx if ldx is not None else x.stride(0)
    p.Y, p.ldy = y.data_ptr(), ldy if ldy is not None else y.stride(0)
    p.bias, p.residual = ptr(bias), ptr(residual)
    p.ld_res = ld_res if ld_res is not None else (residual.stride(0) if residual is not None else 0)
    p.act, p.splitk = act, splitk
    p.flags = (GM_OUT_BF16 if y.dtype == torch.bfloat16 else 0) | (GM_RES_MUL if res_mul else 0)
    p._pad = wide                       # 0: kernel decides between 128- and 256-row CTAs (m > 128), 1: 128 rows, 2: 256 rows
    return p


def gemm_plan(p: S.GemmParams):
    """(tokens per CTA, weight rows per CTA, K splits) the launcher will use for this description."""
    nt, rows, sk = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    check(lib().rlz_gemm_plan(ctypes.byref(p), ctypes.byref(nt), ctypes.byref(rows), ctypes.byref(sk)), "gemm_plan")
    return nt.value, rows.value, sk.value


def gemm_launch(p: S.GemmParams) -> None:
    check(lib().rlz_gemm_kquant(ctypes.byref(p), stream_ptr()), "gemm_kquant")


def gemm(w: DeviceWeight, x: torch.Tensor, bias=None, residual=None, act=ACT_NONE, splitk: Optional[int] = None) -> torch.Tensor:
    """Convenience form: allocates the output.  With split-K the output starts as the residual (or
    zeros) and the partial products are accumulated atomically."""
    x2 = x.reshape(-1, w.k).to(torch.bfloat16).contiguous()
    m = x2.shape[0]
    sk = splitk if splitk is not None else (choose_splitk(w.n, w.k, m) if act == ACT_NONE else 1)
    if sk > 1:
        y = residual.reshape(m, w.n).float().clone() if residual is not None else torch.zeros(m, w.n, device=x.device, dtype=torch.float32)
        gemm_launch(build_gemm_params(w, x2, y, m, bias=bias, splitk=sk))
    else:
        y = torch.empty(m, w.n, device=x.device, dtype=torch.float32)
        res = residual.reshape(m, w.n).float().contiguous() if residual is not None else None
        gemm_launch(build_gemm_params(w, x2, y, m, bias=bias, residual=res, act=act))
    return y.reshape(*x.shape[:-1], w.n)


class GemmPlan:
    """Reusable launch of one weight matrix at a fixed token count (micro-benchmarks)."""

    def __init__(self, w: DeviceWeight, m: int, device, splitk: Optional[int] = None, wide: int = 0):
        self.w, self.m, self.wide = w, m, wide
        self.splitk = splitk if splitk is not None else choose_splitk(w.n, w.k, m)

    def run(self, x: torch.Tensor, y: torch.Tensor) -> None:
        if self.splitk > 1:
            y.zero_()
        gemm_launch(build_gemm_params(self.w, x, y, self.m, splitk=self.splitk, wide=self.wide))
