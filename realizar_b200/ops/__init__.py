"""Python entry points of the sm_100a kernels (``librlz_cuda.so``).

Every wrapper launches on the current torch CUDA stream, so calls compose with torch ops and
can be captured into CUDA graphs.  There is no fallback implementation: if the native library
is missing on a GPU host the import of :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .._native import cuda_lib
from ..quant import QType
from ..quant.device_layout import dev_row_bytes, to_device_layout
from . import _signatures as S
from ._signatures import (ACT_GELU, ACT_NONE, ACT_SILU, COMBINE_ADD, COMBINE_GELU_MUL, COMBINE_SILU_MUL, NORM_LAYER,
                          NORM_NONE, NORM_RMS)


class KernelError(RuntimeError):
    pass


def lib():
    return cuda_lib()


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc > 0:
        msg = lib().rlz_cuda_error_string(rc).decode()
        raise KernelError(f"{what}: CUDA error {rc} ({msg})")
    raise KernelError(f"{what}: invalid arguments (code {rc})")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def launch_count() -> int:
    return int(lib().rlz_launch_count())


def set_pdl(on: bool) -> None:
    lib().rlz_set_pdl(1 if on else 0)


# ------------------------------------------------------------------------------ weights ----
@dataclass
class DeviceWeight:
    """A weight matrix resident on the GPU in the device layout of its block type."""
    data: torch.Tensor      # uint8 [n, stride]
    qtype: int
    n: int
    k: int

    @property
    def stride(self) -> int:
        return self.data.stride(0)

    @property
    def nbytes(self) -> int:
        return self.data.numel()

    def rows(self, r0: int, r1: int) -> "DeviceWeight":
        return DeviceWeight(self.data[r0:r1], self.qtype, r1 - r0, self.k)


def upload_weight(data, qtype: int, n: int, k: int, device) -> DeviceWeight:
    """Stored block bytes (numpy or torch uint8, flat) -> device layout on ``device``."""
    t = data if isinstance(data, torch.Tensor) else torch.from_numpy(data)
    t = t.to(device, non_blocking=True).reshape(-1)
    dev = to_device_layout(t, qtype, n, k).contiguous()
    assert dev.shape == (n, dev_row_bytes(qtype, k)), (dev.shape, n, dev_row_bytes(qtype, k))
    return DeviceWeight(dev, int(qtype), n, k)


# ------------------------------------------------------------------------------ GEMV -------
@dataclass
class VecIn:
    """Input vector(s) ``[batch, k]`` (row stride ``ld``) with an optional fused norm."""
    x: torch.Tensor
    k: int
    ld: Optional[int] = None
    norm: int = NORM_NONE
    norm_w: Optional[torch.Tensor] = None
    norm_b: Optional[torch.Tensor] = None
    eps: float = 1e-5
    pre: Optional[torch.Tensor] = None     # batch 1: the int8 activation block written by the producing launch (MatOut.q_out)


def act_block_bytes(k: int) -> int:
    """Bytes of a pre-quantised activation block of ``k`` values: codes, per-64 records, per-32 scales, per-16 sums."""
    return k + k // 4 + k // 8 + k // 4


@dataclass
class MatOut:
    """A block of output rows: one or two (weight, input index) pairs and an epilogue."""
    segs: Sequence[tuple]                  # [(DeviceWeight, x_index), ...]
    out_off: int = 0
    bias: Optional[torch.Tensor] = None
    bias2: Optional[torch.Tensor] = None
    combine: int = COMBINE_ADD
    act: int = ACT_NONE
    residual: bool = False
    rows_per_cta: int = 0                  # 0 = choose automatically
    q_out: Optional[torch.Tensor] = None   # batch 1: also write the outputs as the int8 activation block of the next launch
    q_out_k: int = 0                       # length of that activation vector
    q_out_col0: int = 0                    # column of this matrix's row 0 in it


def plan_rows_per_cta(mats: Sequence[MatOut], target_ctas: int) -> List[int]:
    """Rows per CTA of every matrix of a launch: the smallest per-CTA byte budget for which the launch needs at most
    ``target_ctas`` CTAs (one wave), so that every CTA streams about the same number of weight bytes.  Matrices that
    also write their outputs as an int8 block hand out rows in multiples of 32 (one quantisation block per warp)."""
    n = [m.segs[0][0].n for m in mats]
    rowb = [max(1.0, sum(w.nbytes for w, _ in m.segs) / max(1, ni)) for m, ni in zip(mats, n)]
    gran = [32 if m.q_out is not None else 1 for m in mats]

    def rows_for(budget: float, i: int) -> int:
        return min(1024, max(gran[i], int(budget / rowb[i]) // gran[i] * gran[i]))

    def ctas_for(budget: float) -> int:
        return sum(-(-n[i] // rows_for(budget, i)) for i in range(len(mats)))

    lo, hi = 1.0, max(rb * ni for rb, ni in zip(rowb, n)) + 1.0
    if ctas_for(hi) > target_ctas:                     # more matrices than CTAs, or rows capped at 1024: one CTA each at least
        return [rows_for(hi, i) for i in range(len(mats))]
    for _ in range(48):
        mid = 0.5 * (lo + hi)
        if ctas_for(mid) <= target_ctas:
            hi = mid
        else:
            lo = mid
    out = []
    for i in range(len(mats)):
        ctas = -(-n[i] // rows_for(hi, i))
        out.append(min(1024, max(gran[i], -(-(-(-n[i] // ctas)) // gran[i]) * gran[i])))    # same CTA count, rows evened out
    return out


def build_gemv_params(xs: Sequence[VecIn], mats: Sequence[MatOut], y: torch.Tensor, batch: int, ldy: Optional[int] = None,
                      residual: Optional[torch.Tensor] = None, ld_res: Optional[int] = None, target_ctas: int = 148,
                      ar: Optional[S.GemvAr] = None) -> S.GemvParams:
    """Fill a parameter block.  The caller keeps every referenced tensor alive."""
    if not (1 <= len(mats) <= S.GEMV_MAX_MATS and 1 <= len(xs) <= S.GEMV_MAX_X):
        raise ValueError("a GEMV launch takes 1..4 matrices and 1..4 inputs")
    p = S.GemvParams()
    auto = plan_rows_per_cta(mats, target_ctas)
    for i, v in enumerate(xs):
        X = p.xs[i]
        X.x, X.nw, X.nb = v.x.data_ptr(), ptr(v.norm_w), ptr(v.norm_b)
        X.ld = v.ld if v.ld is not None else v.x.stride(0) if v.x.dim() > 1 else v.k
        X.k, X.norm, X.eps = v.k, v.norm, v.eps
        if v.pre is not None:
            if batch != 1 or v.norm != NORM_NONE or v.k % 128 or v.pre.numel() < act_block_bytes(v.k):
                raise ValueError("a pre-quantised input needs batch 1, no norm, k % 128 == 0 and a block of act_block_bytes(k)")
            X.pre = v.pre.data_ptr()
    for i, m in enumerate(mats):
        M = p.mat[i]
        M.nseg = len(m.segs)
        for s, (w, xi) in enumerate(m.segs):
            seg = M.seg[s]
            seg.W, seg.stride, seg.qtype, seg.k, seg.x_id = w.data.data_ptr(), w.stride, w.qtype, w.k, xi
            if xs[xi].k != w.k:
                raise ValueError(f"matrix {i} segment {s}: k={w.k} but input {xi} has k={xs[xi].k}")
        M.bias, M.bias2 = ptr(m.bias), ptr(m.bias2)
        M.combine, M.act, M.has_residual = m.combine, m.act, 1 if m.residual else 0
        M.n, M.out_off = m.segs[0][0].n, m.out_off
        M.rows_per_cta = m.rows_per_cta or auto[i]
        if m.q_out is not None:
            if batch != 1:
                raise ValueError("quantised output is a batch-1 feature")
            M.rows_per_cta = -(-M.rows_per_cta // 32) * 32        # a warp of the epilogue owns one 32-value quantisation block (explicit rows_per_cta)
            M.q_out, M.q_out_k, M.q_out_col0 = m.q_out.data_ptr(), m.q_out_k, m.q_out_col0
    p.nmat, p.batch = len(mats), batch
    p.y, p.ldy = y.data_ptr(), ldy if ldy is not None else (y.stride(0) if y.dim() > 1 else y.numel())
    p.residual = ptr(residual)
    p.ld_res = ld_res if ld_res is not None else (residual.stride(0) if residual is not None and residual.dim() > 1 else 0)
    if ar is not None:
        ctypes.memmove(ctypes.addressof(p.ar), ctypes.addressof(ar), ctypes.sizeof(S.GemvAr))
    return p


def slab_eligible(p: S.GemvParams) -> bool:
    """True when the launch can run on the copy-engine-fed GEMV (``csrc/kernels/gemv_slab.cu``): K-quant rows with
    k % 256 == 0 whose activations plus one pass per warp fit half an SM's shared memory.  ``RLZ_GEMV_SLAB=0`` keeps
    every launch on the register-path kernel (kernel comparisons)."""
    if os.environ.get("RLZ_GEMV_SLAB", "1") == "0":
        return False
    return int(lib().rlz_gemv_slab_check(ctypes.byref(p))) == 0


def gemv_launch(p: S.GemvParams) -> None:
    """Launch a prepared GEMV description on the kernel that takes it (decided once per description)."""
    slab = getattr(p, "_slab", None)
    if slab is None:
        slab = p._slab = slab_eligible(p)
    if slab:
        check(lib().rlz_gemv_slab(ctypes.byref(p), stream_ptr()), "gemv_slab")
    else:
        check(lib().rlz_gemv(ctypes.byref(p), stream_ptr()), "gemv")


STREAM_TYPES = (int(QType.Q4_K), int(QType.Q5_K), int(QType.Q6_K))


def stream_eligible(mats: Sequence[MatOut]) -> bool:
    """True when every matrix of a launch can go through the TMA-streamed GEMV kernel."""
    if os.environ.get("RLZ_GEMV_STREAM", "0") != "1":       # opt-in: the register-path kernel measures faster at decode sizes
        return False
    for m in mats:
        for w, _ in m.segs:
            if w.qtype not in STREAM_TYPES or w.k % 256 or w.stride != dev_row_bytes(w.qtype, w.k):
                return False
    return True


def gemv_stream_launch(p: S.GemvParams) -> None:
    check(lib().rlz_gemv_stream(ctypes.byref(p), stream_ptr()), "gemv_stream")


def device_error(clear: bool = True) -> int:
    """Error code recorded by a kernel whose bounded wait expired (0 = none)."""
    c = 1 if clear else 0
    return (int(lib().rlz_device_error(c)) or int(lib().rlz_gemv_slab_error(c)) or int(lib().rlz_gemm_error(c))
            or int(lib().rlz_attn_decode_error(c)) or int(lib().rlz_attn_prefill_error(c)) or int(lib().rlz_index_error(c)))


def gemv(w: DeviceWeight, x: torch.Tensor, bias=None, act=ACT_NONE, residual=None, norm=NORM_NONE, norm_w=None, norm_b=None,
         eps=1e-5, stream: Optional[bool] = None) -> torch.Tensor:
    """``y = act(W norm(x) + bias) + residual`` for ``x`` of shape ``[batch<=4, k]`` (convenience form)."""
    x2 = x.reshape(-1, w.k).contiguous().float()
    batch = x2.shape[0]
    y = torch.empty(batch, w.n, device=x.device, dtype=torch.float32)
    res = residual.reshape(batch, w.n).contiguous().float() if residual is not None else None
    mats = [MatOut([(w, 0)], bias=bias, act=act, residual=res is not None)]
    use_stream = stream_eligible(mats) if stream is None else stream
    p = build_gemv_params([VecIn(x2, w.k, norm=norm, norm_w=norm_w, norm_b=norm_b, eps=eps)], mats, y, batch, residual=res,
                          target_ctas=148)
    (gemv_stream_launch if use_stream else gemv_launch)(p)
    return y.reshape(*x.shape[:-1], w.n)


# ------------------------------------------------------------------------------ attention --
def attn_decode_scratch(batch: int, n_heads: int, splits: int, head_dim: int, device):
    partial = torch.empty(int(lib().rlz_attn_decode_partial_floats(batch, n_heads, splits, head_dim)), device=device, dtype=torch.float32)
    counters = torch.zeros(int(lib().rlz_attn_decode_counter_ints(batch, n_heads)), device=device, dtype=torch.int32)
    return partial, counters


def build_attn_decode_params(qkv, out, k_cache, v_cache, positions, page_table, partial, counters, n_heads, n_kv_heads, head_dim,
                             splits, batch, rope_dim, rope_type, rope_theta, q_off, k_off, v_off, q_norm_w=None, k_norm_w=None,
                             eps=1e-6, ld_qkv=None, ld_out=None, shared_table=False, no_append=False, window=0, rope_table=None) -> S.AttnDecodeParams:
    p = S.AttnDecodeParams()
    p.qkv, p.out, p.k_cache, p.v_cache = qkv.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    p.positions, p.page_table = positions.data_ptr(), page_table.data_ptr()
    p.q_norm_w, p.k_norm_w = ptr(q_norm_w), ptr(k_norm_w)
    p.partial, p.counters = partial.data_ptr(), counters.data_ptr()
    p.ld_qkv = ld_qkv if ld_qkv is not None else qkv.stride(0)
    p.ld_out = ld_out if ld_out is not None else out.stride(0)
    p.n_heads, p.n_kv_heads, p.head_dim, p.max_pages = n_heads, n_kv_heads, head_dim, page_table.shape[-1]
    p.rope_dim, p.rope_type, p.splits, p.batch = rope_dim, rope_type, splits, batch
    p.q_off, p.k_off, p.v_off = q_off, k_off, v_off
    p.rope_theta, p.eps, p.scale = rope_theta, eps, head_dim ** -0.5
    p.pt_stride = 0 if shared_table else (page_table.stride(0) if page_table.dim() > 1 else page_table.shape[-1])
    p.no_append = 1 if no_append else 0
    p.window = int(window or 0)
    p.kv_q8 = 1 if k_cache.dtype in (torch.uint8, torch.int8) else 0
    p.num_pages = int(k_cache.shape[0]) if k_cache.dim() >= 4 else 0      # [pages, kv_heads, page, row]: page ids are checked on the device
    if rope_table is not None:
        if rope_table.dtype != torch.float32 or rope_table.dim() != 3 or rope_table.shape[1] != rope_dim // 2 or rope_table.shape[2] != 2 or not rope_table.is_contiguous():
            raise ValueError("rope_table must be a contiguous float32 [positions, rope_dim / 2, 2] (cos, sin) tensor")
        p.rope_table, p.rope_table_len = rope_table.data_ptr(), rope_table.shape[0]
    return p


def make_rope_table(max_positions: int, rope_dim: int, theta: float, device) -> torch.Tensor:
    """(cos, sin) of ``pos * theta^(-2i/rope_dim)`` for every position and rotary pair, computed in float64."""
    i = torch.arange(rope_dim // 2, dtype=torch.float64)
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rope_dim)[None, :]
    return torch.stack([ang.cos(), ang.sin()], -1).to(torch.float32).contiguous().to(device)


def attn_decode_launch(p: S.AttnDecodeParams) -> None:
    check(lib().rlz_attn_decode(ctypes.byref(p), stream_ptr()), "attn_decode")


def attn_prefill_supported(head_dim: int) -> bool:
    return bool(lib().rlz_attn_prefill_supported(int(head_dim)))


def attn_prefill(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, n_tokens: int,
                 pos0: int, n_heads: int, n_kv_heads: int, head_dim: int, q_off: int = 0, window: int = 0,
                 pos0_dev: Optional[torch.Tensor] = None, impl: Optional[str] = None) -> None:
    """Causal attention of chunk rows ``pos0 .. pos0+n_tokens-1`` of one sequence over its paged cache
    (tensor-core kernel; the chunk's own K/V rows must already be in the cache).  With ``pos0_dev`` (an int32 device
    tensor) the position of row 0 is read on the device, so a captured launch serves every chunk position.
    ``impl``: "tc" (128-query tiles on tcgen05) or "mma" (16-query tiles on mma.sync); None = the launcher's choice."""
    p = S.AttnPrefillParams()
    p.qkv, p.out, p.k_cache, p.v_cache, p.page_table = qkv.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr()
    p.ld_qkv, p.ld_out = qkv.stride(0), out.stride(0)
    p.n_heads, p.n_kv_heads, p.head_dim, p.q_off = n_heads, n_kv_heads, head_dim, q_off
    p.n_tokens, p.pos0, p.window, p.scale = int(n_tokens), int(pos0), int(window or 0), head_dim ** -0.5
    p.kv_q8 = 1 if k_cache.dtype in (torch.uint8, torch.int8) else 0
    p.out_bf16 = 1 if out.dtype == torch.bfloat16 else 0          # bf16: written as the operand of the output-projection GEMM
    p.pos0_ptr = ptr(pos0_dev)
    check(lib().rlz_attn_prefill_impl(ctypes.byref(p), stream_ptr(), {None: -1, "tc": 0, "mma": 1}[impl]), "attn_prefill")


def attn_prefill_error(clear: bool = True) -> int:
    return int(lib().rlz_attn_prefill_error(1 if clear else 0))


def kv_cache_alloc(layers: int, pages: int, kv_heads: int, head_dim: int, device, dtype: str = "bf16", page: int = 16) -> torch.Tensor:
    """``[2 (k, v), layers, pages, kv_heads, page, row]``: bf16 rows of ``head_dim``, or with ``dtype="q8"`` uint8 rows of
    ``head_dim + 16`` bytes (int8 codes, the fp32 scale of the row, padding)."""
    if dtype == "q8":
        return torch.zeros(2, layers, pages, kv_heads, page, head_dim + 16, device=device, dtype=torch.uint8)
    if dtype != "bf16":
        raise ValueError(f"unknown KV cache dtype '{dtype}' (bf16 | q8)")
    return torch.zeros(2, layers, pages, kv_heads, page, head_dim, device=device, dtype=torch.bfloat16)


def kv_rows_to_float(cache: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Decode cache rows ``[..., row]`` (either layout) to fp32 ``[..., head_dim]`` (tests, snapshots, debugging)."""
    if cache.dtype == torch.bfloat16:
        return cache.float()
    codes = cache[..., :head_dim].contiguous().view(torch.int8).float()
    scale = cache[..., head_dim:head_dim + 4].contiguous().view(torch.float32)
    return codes * scale


# ------------------------------------------------------------------------------ small ops --
def embed(table: torch.Tensor, qtype: int, row_bytes: int, hidden: int, vocab: int, tokens: torch.Tensor, out: torch.Tensor,
          pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> None:
    check(lib().rlz_embed(table.data_ptr(), int(qtype), row_bytes, hidden, vocab, tokens.data_ptr(), tokens.numel(), ptr(pos_table),
                          ptr(positions), out.data_ptr(), out.stride(0), stream_ptr()), "embed")


def norm(x: torch.Tensor, w=None, b=None, norm_type=NORM_RMS, eps=1e-5, residual=None, sum_out=None) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    y = torch.empty_like(x2)
    check(lib().rlz_norm(x2.data_ptr(), ptr(residual), ptr(w), ptr(b), y.data_ptr(), ptr(sum_out), x2.shape[0], x2.shape[1], x2.stride(0),
                         norm_type, eps, stream_ptr()), "norm")
    return y.reshape(x.shape)


def head_rmsnorm_(x: torch.Tensor, w: torch.Tensor, heads: int, d: int, eps: float) -> None:
    check(lib().rlz_head_rmsnorm(x.data_ptr(), w.data_ptr(), x.shape[0], heads, d, x.stride(0), eps, stream_ptr()), "head_rmsnorm")


def rope_(x: torch.Tensor, positions: torch.Tensor, heads: int, d: int, rope_dim: int, rope_type: int, theta: float,
          table: Optional[torch.Tensor] = None) -> None:
    """In-place RoPE on ``x [T, >= heads*d]`` (row stride taken from the tensor).  ``table``: ``[positions, rope_dim/2, 2]``
    (cos, sin) as made by ``make_rope_table`` - carries the checkpoint's context scaling; positions beyond it use ``theta``."""
    check(lib().rlz_rope(x.data_ptr(), positions.data_ptr(), x.shape[0], heads, d, x.stride(0), rope_dim, rope_type, theta,
                         ptr(table), int(table.shape[0]) if table is not None else 0, stream_ptr()), "rope")


def elementwise(a: torch.Tensor, b=None, bias=None, residual=None, act=ACT_NONE, out=None) -> torch.Tensor:
    """``act(a + bias) [* b] [+ residual]`` over 2-D views."""
    a2 = a.reshape(-1, a.shape[-1])
    y = out if out is not None else torch.empty(a2.shape, device=a.device, dtype=torch.float32)
    y2 = y.reshape(-1, y.shape[-1])
    b2 = b.reshape(-1, b.shape[-1]) if b is not None else None
    check(lib().rlz_elementwise(a2.data_ptr(), ptr(b2), ptr(bias), ptr(residual), y2.data_ptr(), a2.shape[0], a2.shape[1], a2.stride(0),
                                b2.stride(0) if b2 is not None else 0, y2.stride(0), act, 1 if b is not None else 0, stream_ptr()), "elementwise")
    return y.reshape(a.shape) if out is None else y


def to_bf16(src: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 [rows, cols] -> bf16 (own kernel; row strides taken from the tensors)."""
    s2 = src.reshape(-1, src.shape[-1])
    if out is None:
        out = torch.empty(s2.shape, device=src.device, dtype=torch.bfloat16)
    check(lib().rlz_to_bf16(s2.data_ptr(), out.data_ptr(), s2.shape[0], s2.shape[1], s2.stride(0), out.stride(0), stream_ptr()), "to_bf16")
    return out


def norm_bf16(x: torch.Tensor, out: torch.Tensor, w=None, b=None, norm_type=NORM_RMS, eps=1e-5) -> torch.Tensor:
    """``out = bf16(norm(x))`` for 2-D ``x`` (one launch: the GEMM operand producer of prefill)."""
    check(lib().rlz_norm_bf16(x.data_ptr(), ptr(w), ptr(b), out.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.stride(0), norm_type, eps,
                              stream_ptr()), "norm_bf16")
    return out


def swiglu_bf16(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor, act=ACT_SILU) -> torch.Tensor:
    """``out = bf16(act(gate) * up)`` (``up`` may be None: plain activation)."""
    check(lib().rlz_swiglu_bf16(gate.data_ptr(), ptr(up), out.data_ptr(), gate.shape[0], gate.shape[1], gate.stride(0),
                                up.stride(0) if up is not None else 0, out.stride(0), act, stream_ptr()), "swiglu_bf16")
    return out


def kv_append(k, v, k_cache, v_cache, positions, page_rows, n_kv_heads, d, page=16) -> None:
    """Write the rows of ``k`` / ``v`` at their positions into the paged cache (bf16 rows, or int8 rows with a per-row scale)."""
    fn = lib().rlz_kv_append_q8 if k_cache.dtype in (torch.uint8, torch.int8) else lib().rlz_kv_append
    check(fn(k.data_ptr(), v.data_ptr(), k.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
             page_rows.data_ptr(), k.shape[0], n_kv_heads, d, page, k_cache.shape[0], stream_ptr()), "kv_append")


def page_rows(page_table: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n: int, page: int) -> None:
    check(lib().rlz_page_rows(page_table.data_ptr(), page_table.stride(0), positions.data_ptr(), out.data_ptr(), n, page, stream_ptr()), "page_rows")


def advance_(tokens: torch.Tensor, sampled: torch.Tensor, positions: torch.Tensor, limit: int = 0) -> None:
    """Device-side feedback: sampled ids become the next inputs and positions move on.  With ``limit`` > 0 a sequence
    whose next position would reach ``limit`` (the length its KV pages were reserved for) goes idle (position -1)
    instead of running past its page table."""
    check(lib().rlz_advance(tokens.data_ptr(), sampled.data_ptr(), positions.data_ptr(), tokens.numel(), int(limit), stream_ptr()), "advance")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, out_val: Optional[torch.Tensor] = None, index_offset: int = 0,
           vocab: Optional[int] = None) -> torch.Tensor:
    l2 = logits.reshape(-1, logits.shape[-1])
    if out is None:
        out = torch.empty(l2.shape[0], device=logits.device, dtype=torch.int32)
    check(lib().rlz_argmax(l2.data_ptr(), l2.stride(0), vocab or l2.shape[1], l2.shape[0], out.data_ptr(), ptr(out_val), index_offset, stream_ptr()), "argmax")
    return out


def build_sample_params(logits, temperature, top_k, top_p, uniform, out, min_p=None, out_logprob=None, vocab=None) -> S.SampleParams:
    p = S.SampleParams()
    l2 = logits.reshape(-1, logits.shape[-1])
    p.logits, p.ld, p.vocab, p.batch = l2.data_ptr(), l2.stride(0), vocab or l2.shape[1], l2.shape[0]
    p.temperature, p.top_k, p.top_p, p.min_p = temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), ptr(min_p)
    p.uniform, p.out, p.out_logprob = uniform.data_ptr(), out.data_ptr(), ptr(out_logprob)
    return p


def sample_launch(p: S.SampleParams) -> None:
    check(lib().rlz_sample(ctypes.byref(p), stream_ptr()), "sample")


def sample(logits, temperature, top_k, top_p, uniform, min_p=None) -> torch.Tensor:
    out = torch.empty(logits.reshape(-1, logits.shape[-1]).shape[0], device=logits.device, dtype=torch.int32)
    sample_launch(build_sample_params(logits, temperature, top_k, top_p, uniform, out, min_p))
    return out


def history_push(history: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, batch: int) -> None:
    """``history[b, positions[b] % window] = tokens[b]`` for the active rows (the ring the penalties read)."""
    check(lib().rlz_history_push(history.data_ptr(), history.shape[-1], tokens.data_ptr(), positions.data_ptr(), batch, stream_ptr()), "history_push")


def logit_controls(logits: torch.Tensor, history, repetition, presence, frequency, bias, bias_on, index_offset: int = 0,
                   vocab: Optional[int] = None) -> None:
    """In place, per row: additive bias / mask row (rows with ``bias_on``) and repetition / presence / frequency penalties."""
    l2 = logits.reshape(-1, logits.shape[-1])
    check(lib().rlz_logit_controls(l2.data_ptr(), l2.stride(0), vocab or l2.shape[1], index_offset, l2.shape[0], ptr(history),
                                   history.shape[-1] if history is not None else 1, ptr(repetition), ptr(presence), ptr(frequency), ptr(bias),
                                   bias.stride(0) if bias is not None else 0, ptr(bias_on), stream_ptr()), "logit_controls")


def logprob_parts(logits: torch.Tensor, targets: torch.Tensor, index_offset: int = 0, vocab: Optional[int] = None) -> torch.Tensor:
    """Per row of ``logits`` ``[rows, >= vocab]``: ``[max, sum exp(logit - max), logit[target - index_offset] or -inf]`` (fp32 ``[rows, 3]``).
    With one vocabulary slice ``log p(target) = out[:, 2] - out[:, 0] - log(out[:, 1])``."""
    l2 = logits.reshape(-1, logits.shape[-1])
    out = torch.empty(l2.shape[0], 3, device=logits.device, dtype=torch.float32)
    check(lib().rlz_logprob_rows(l2.data_ptr(), l2.stride(0), vocab or l2.shape[1], l2.shape[0], targets.data_ptr(), index_offset, out.data_ptr(),
                                 stream_ptr()), "logprob_rows")
    return out


def penalties_(logits, history, repetition=None, presence=None, frequency=None) -> None:
    l2 = logits.reshape(-1, logits.shape[-1])
    check(lib().rlz_penalties(l2.data_ptr(), l2.stride(0), l2.shape[1], l2.shape[0], history.data_ptr(), history.shape[-1], ptr(repetition),
                              ptr(presence), ptr(frequency), stream_ptr()), "penalties")
