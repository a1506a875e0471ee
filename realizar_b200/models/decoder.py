"""GPU decoder: uploads a ``ModelWeights`` to one GPU (optionally a tensor-parallel shard of
it) and builds the per-step launch plan of the decode kernels.

Launch plan for one decode step of ``batch`` sequences (L layers):

* sequential-residual models (Llama / Qwen2 / Mistral ...), 5 launches per layer:
  ``gemv[attn_norm -> Q|K|V (+bias)]`` -> ``attn_decode[qk-norm, rope, kv append, flash-decode]``
  -> ``gemv[o_proj + residual]`` -> ``gemv[ffn_norm -> silu(gate) * up]`` -> ``gemv[down + residual]``
* parallel-residual models (Phi-2), 3 launches per layer:
  ``gemv[layernorm -> QKV (+bias) | gelu(fc1 + bias)]`` -> ``attn_decode`` ->
  ``gemv[o_proj(attn) + fc2(act) + biases + residual]``
* then ``gemv[output_norm -> lm_head]`` and the token selection kernel.

The reference's equivalent is ``transformer_layer_workspace_inner`` with ~10 launches per layer
(src/cuda/executor/layers/gemv_dispatch.rs:53-309) and its capability gate that keeps
LayerNorm / GELU models off the GPU (src/gguf/cuda/loading.rs:250-270); here they run on the
same kernels.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..ops import (ACT_GELU, ACT_NONE, COMBINE_ADD, COMBINE_GELU_MUL, COMBINE_SILU_MUL, NORM_LAYER, NORM_NONE, NORM_RMS,
                   DeviceWeight, MatOut, VecIn)
from ..quant import BLOCK_SPECS, QType, row_bytes
from .config import ModelConfig
from .weights import ModelWeights, QTensor

log = logging.getLogger(__name__)


def _f32(t: Optional[QTensor], device) -> Optional[torch.Tensor]:
    """Small tensors (norm weights, biases, position table) as contiguous f32 on the device."""
    if t is None:
        return None
    return torch.from_numpy(np.ascontiguousarray(t.to_f32())).to(device)


def shard_rows(t: QTensor, r0: int, r1: int) -> QTensor:
    """Rows [r0, r1) of a stored matrix (column-parallel shard)."""
    n, k = t.shape
    rb = row_bytes(t.qtype, k)
    data = t.data.reshape(-1)[r0 * rb: r1 * rb]
    return QTensor(t.qtype, (r1 - r0, k), data)


def shard_cols(t: QTensor, k0: int, k1: int):
    """Columns [k0, k1) of a stored matrix (row-parallel shard).

    Block types cannot be cut inside a block, so the shard keeps every block that overlaps the
    range and silences the sub-blocks outside it by zeroing their scales (Q4_K / Q5_K: 32-wide,
    Q6_K: 16-wide sub-blocks).  Returns ``(shard, cover_start)``: the shard multiplies the
    activation slice ``[cover_start, cover_start + shard.k)`` whose entries outside ``[k0, k1)``
    must be zero.
    """
    n, k = t.shape
    qt = QType(t.qtype)
    spec = BLOCK_SPECS[qt]
    sub = {QType.Q4_K: 32, QType.Q5_K: 32, QType.Q6_K: 16}.get(qt, spec.elems)
    if k0 % sub or k1 % sub:
        raise ValueError(f"{qt.name} weights can only be split at multiples of {sub} columns (got {k0}:{k1})")
    b0, b1 = k0 // spec.elems, -(-k1 // spec.elems)
    data = t.data if isinstance(t.data, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(t.data))
    blocks = data.reshape(n, k // spec.elems, spec.nbytes)[:, b0:b1].clone()
    cover0 = b0 * spec.elems
    if spec.elems == 256:
        for bi, blk in ((0, b0), (blocks.shape[1] - 1, b1 - 1)):
            lo, hi = blk * 256, blk * 256 + 256
            for j in range(256 // sub):
                s0 = lo + j * sub
                if s0 >= k0 and s0 + sub <= k1:
                    continue
                if qt == QType.Q6_K:
                    blocks[:, bi, 192 + j] = 0
                else:                       # packed 6-bit scale / min of sub-block j
                    sc = blocks[:, bi, 4:16]
                    if j < 4:
                        sc[:, j] &= 0xC0
                        sc[:, j + 4] &= 0xC0
                    else:
                        sc[:, j + 4] = 0
                        sc[:, j - 4] &= 0x3F
                        sc[:, j] &= 0x3F
    out = QTensor(t.qtype, (n, (b1 - b0) * spec.elems), blocks.reshape(-1))
    return out, cover0


@dataclass
class LayerWeights:
    attn_norm_w: Optional[torch.Tensor] = None
    attn_norm_b: Optional[torch.Tensor] = None
    ffn_norm_w: Optional[torch.Tensor] = None
    ffn_norm_b: Optional[torch.Tensor] = None
    q: Optional[DeviceWeight] = None
    k: Optional[DeviceWeight] = None
    v: Optional[DeviceWeight] = None
    q_b: Optional[torch.Tensor] = None
    qkv: Optional[DeviceWeight] = None     # Q, K, V as one matrix (their rows are views of it) when they share a block type
    qkv_b: Optional[torch.Tensor] = None
    k_b: Optional[torch.Tensor] = None
    v_b: Optional[torch.Tensor] = None
    o: Optional[DeviceWeight] = None
    o_b: Optional[torch.Tensor] = None
    gate: Optional[DeviceWeight] = None
    up: Optional[DeviceWeight] = None
    up_b: Optional[torch.Tensor] = None
    down: Optional[DeviceWeight] = None
    down_b: Optional[torch.Tensor] = None
    q_norm_w: Optional[torch.Tensor] = None
    k_norm_w: Optional[torch.Tensor] = None
    o_in_off: int = 0          # offset of this rank's attention output inside the o_proj input buffer
    down_in_off: int = 0       # same for the MLP activation inside the down-proj input buffer


def make_rope_table(cfg, device, max_positions: Optional[int] = None) -> torch.Tensor:
    """(cos, sin) per position and rotary pair, with the checkpoint's context scaling
    (linear / NTK / YaRN; src/layers ``ScaledRoPE`` in the reference) folded in."""
    from .layers import RoPE, RopeScaling, RopeScalingType
    n = max_positions or min(cfg.context_length, 1 << 17)
    kind = {"linear": RopeScalingType.LINEAR, "ntk": RopeScalingType.NTK, "yarn": RopeScalingType.YARN}.get(str(cfg.rope_scaling_type).lower())
    if kind is None or cfg.rope_scaling_factor == 1.0:
        return ops.make_rope_table(n, cfg.rope_dim, cfg.rope_theta, device)
    inv, mscale = RoPE(cfg.rope_dim, cfg.rope_theta, scaling=RopeScaling(kind, cfg.rope_scaling_factor, cfg.rope_original_context or cfg.context_length)).inv_freq(n)
    ang = torch.arange(n, dtype=torch.float64)[:, None] * inv.double()[None, :]
    return torch.stack([ang.cos() * mscale, ang.sin() * mscale], -1).to(torch.float32).contiguous().to(device)


class GpuModel:
    """Weights of one (shard of a) decoder on one GPU."""

    def __init__(self, weights: ModelWeights, device="cuda", tp_rank: int = 0, tp_size: int = 1, resident_layers: Optional[int] = None):
        """``resident_layers``: keep only the first that many layers' matrices on the device; the others stay in pinned host
        memory and are streamed through two device buffers while the model runs (models larger than the device)."""
        cfg = weights.config
        self.cfg = cfg
        self.streamed_from = cfg.num_layers                  # first layer whose matrices are streamed (= num_layers: none)
        self._stream: Dict[int, dict] = {}
        self.device = torch.device(device)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        if cfg.num_heads % tp_size or cfg.num_kv_heads % tp_size or cfg.intermediate_dim % tp_size:
            raise ValueError(f"tensor parallel size {tp_size} must divide heads ({cfg.num_heads}), kv heads "
                             f"({cfg.num_kv_heads}) and the FFN width ({cfg.intermediate_dim})")
        self.heads = cfg.num_heads // tp_size
        self.kv_heads = cfg.num_kv_heads // tp_size
        self.q_dim, self.kv_dim = self.heads * cfg.head_dim, self.kv_heads * cfg.head_dim
        self.inter = cfg.intermediate_dim // tp_size
        # column of the MLP activation inside the qkv|act buffer of parallel-residual models; under TP
        # the activation slice is surrounded by zero padding because row-parallel shards read whole blocks
        self.act_col0 = self.q_dim + 2 * self.kv_dim + (256 if tp_size > 1 else 0)
        dev = self.device
        up = lambda t: ops.upload_weight(t.data, t.qtype, t.shape[0], t.shape[1], dev)

        def up_group(parts):
            """Upload Q, K, V.  When they share a block type and width they become row ranges of ONE device matrix, so
            that the token-batch path can run the three projections as a single GEMM (returns q, k, v, fused-or-None)."""
            if len({(int(t.qtype), t.shape[1]) for t in parts}) != 1:
                return (*[up(t) for t in parts], None)
            flat = [t.data if isinstance(t.data, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(t.data)) for t in parts]
            rows = [t.shape[0] for t in parts]
            fused = ops.upload_weight(torch.cat([f.reshape(-1) for f in flat]), parts[0].qtype, sum(rows), parts[0].shape[1], dev)
            r1, r2 = rows[0], rows[0] + rows[1]
            return fused.rows(0, r1), fused.rows(r1, r2), fused.rows(r2, r2 + rows[2]), fused

        emb = weights["token_embd.weight"]
        self.embed_qtype = int(emb.qtype)
        self.embed_row_bytes = row_bytes(emb.qtype, cfg.hidden_dim)
        self.embed_table = emb.torch_bytes(dev).contiguous()
        pe = weights.get("token_pos_embd.weight")
        self.pos_table = _f32(pe, dev)
        self.rope_table = None
        if cfg.uses_rope:
            self.rope_table = make_rope_table(cfg, dev)

        out_w = weights.output_weight()
        self.vocab = cfg.vocab_size
        v_per = -(-self.vocab // tp_size)
        self.vocab_start = tp_rank * v_per
        self.vocab_local = max(0, min(self.vocab, self.vocab_start + v_per) - self.vocab_start)
        self.lm_head = up(shard_rows(out_w, self.vocab_start, self.vocab_start + self.vocab_local) if tp_size > 1 else out_w)
        ob = weights.get("output.bias")
        self.lm_head_b = _f32(ob, dev)
        if self.lm_head_b is not None and tp_size > 1:
            self.lm_head_b = self.lm_head_b[self.vocab_start: self.vocab_start + self.vocab_local].contiguous()
        self.out_norm_w = _f32(weights.get("output_norm.weight"), dev)
        self.out_norm_b = _f32(weights.get("output_norm.bias"), dev)

        self.layers: List[LayerWeights] = []
        qd, kvd, hd = cfg.q_dim, cfg.kv_dim, cfg.head_dim
        for l in range(cfg.num_layers):
            p = f"blk.{l}."
            L = LayerWeights()
            g = lambda n: weights.get(p + n)
            L.attn_norm_w, L.attn_norm_b = _f32(g("attn_norm.weight"), dev), _f32(g("attn_norm.bias"), dev)
            L.ffn_norm_w, L.ffn_norm_b = _f32(g("ffn_norm.weight"), dev), _f32(g("ffn_norm.bias"), dev)
            q0, q1 = tp_rank * self.q_dim, (tp_rank + 1) * self.q_dim
            k0, k1 = tp_rank * self.kv_dim, (tp_rank + 1) * self.kv_dim
            if g("attn_qkv.weight") is not None:
                qkv, qkv_b = g("attn_qkv.weight"), _f32(g("attn_qkv.bias"), dev)
                L.q, L.k, L.v, L.qkv = up_group([shard_rows(qkv, q0, q1), shard_rows(qkv, qd + k0, qd + k1), shard_rows(qkv, qd + kvd + k0, qd + kvd + k1)])
                if qkv_b is not None:
                    L.q_b, L.k_b, L.v_b = qkv_b[q0:q1].contiguous(), qkv_b[qd + k0: qd + k1].contiguous(), qkv_b[qd + kvd + k0: qd + kvd + k1].contiguous()
            else:
                L.q, L.k, L.v, L.qkv = up_group([shard_rows(g("attn_q.weight"), q0, q1), shard_rows(g("attn_k.weight"), k0, k1), shard_rows(g("attn_v.weight"), k0, k1)])
                bq, bk, bv = _f32(g("attn_q.bias"), dev), _f32(g("attn_k.bias"), dev), _f32(g("attn_v.bias"), dev)
                L.q_b = bq[q0:q1].contiguous() if bq is not None else None
                L.k_b = bk[k0:k1].contiguous() if bk is not None else None
                L.v_b = bv[k0:k1].contiguous() if bv is not None else None
            L.q_norm_w, L.k_norm_w = _f32(g("attn_q_norm.weight"), dev), _f32(g("attn_k_norm.weight"), dev)
            if L.qkv is not None and any(b is not None for b in (L.q_b, L.k_b, L.v_b)):
                L.qkv_b = torch.cat([b if b is not None else torch.zeros(w.n, device=dev) for b, w in ((L.q_b, L.q), (L.k_b, L.k), (L.v_b, L.v))])
            i0, i1 = tp_rank * self.inter, (tp_rank + 1) * self.inter
            if tp_size > 1:
                o_sh, o_cover = shard_cols(g("attn_output.weight"), q0, q1)
                d_sh, d_cover = shard_cols(g("ffn_down.weight"), i0, i1)
                L.o, L.o_in_off = up(o_sh), q0 - o_cover
                L.down, L.down_in_off = up(d_sh), i0 - d_cover
            else:
                L.o, L.down = up(g("attn_output.weight")), up(g("ffn_down.weight"))
            L.o_b, L.down_b = _f32(g("attn_output.bias"), dev), _f32(g("ffn_down.bias"), dev)
            if tp_size > 1 and tp_rank != 0:       # biases of row-parallel layers are added once
                L.o_b = L.down_b = None
            if cfg.gated_ffn:
                L.gate = up(shard_rows(g("ffn_gate.weight"), i0, i1))
            L.up = up(shard_rows(g("ffn_up.weight"), i0, i1))
            ub = _f32(g("ffn_up.bias"), dev)
            L.up_b = ub[i0:i1].contiguous() if ub is not None else None
            self.layers.append(L)
            if resident_layers is not None and l >= max(0, resident_layers):
                self._offload_layer(l, L)
        if self._stream:
            self._finish_streaming()

    # -- layer streaming: matrices of the later layers live in pinned host memory ------------------------------------------
    # (role of the reference's streaming plan and layer prefetcher, src/cuda/streaming.rs:36-219)
    @staticmethod
    def _layer_mats(L) -> list:
        """The distinct device matrices of a layer (Q, K, V count once when they are row ranges of one matrix)."""
        base = [L.qkv] if L.qkv is not None else [L.q, L.k, L.v]
        return [w for w in base + [L.o, L.gate, L.up, L.down] if w is not None]

    def _offload_layer(self, l: int, L) -> None:
        mats = self._layer_mats(L)
        off, spans = 0, []
        for w in mats:
            spans.append((off, w.data.shape[0], w.data.shape[1]))
            off += (w.data.numel() + 255) // 256 * 256
        from ..runtime.memory import PinnedHostBuffer
        host = PinnedHostBuffer(off).tensor                  # page-locked when the host allows it (copies then overlap with compute)
        for w, (o, n, stride) in zip(mats, spans):
            host[o:o + n * stride].copy_(w.data.reshape(-1))
        qkv_rows = (L.q.n, L.k.n, L.v.n) if L.qkv is not None else None
        for w in mats + ([L.q, L.k, L.v] if L.qkv is not None else []):
            w.data = None                                    # the device copy goes; views are re-created over the stream buffers
        self._stream[l] = {"host": host, "spans": spans, "bytes": off, "qkv_rows": qkv_rows}
        self.streamed_from = min(self.streamed_from, l)

    def _finish_streaming(self) -> None:
        dev = self.device
        size = max(st["bytes"] for st in self._stream.values())
        self._slots = [torch.empty(size, dtype=torch.uint8, device=dev) for _ in range(2)]
        self._slot_layer = [-1, -1]
        self._side = torch.cuda.Stream(dev)
        self._ready = [torch.cuda.Event(), torch.cuda.Event()]
        self._freed = [torch.cuda.Event(), torch.cuda.Event()]
        self._freed_valid = [False, False]
        self.stream_copies = 0
        for l, st in self._stream.items():
            L, buf = self.layers[l], self._slots[(l - self.streamed_from) & 1]
            for w, (o, n, stride) in zip(self._layer_mats(L), st["spans"]):
                w.data = buf[o:o + n * stride].view(n, stride)
            if st["qkv_rows"] is not None:
                r1, r2, r3 = st["qkv_rows"][0], st["qkv_rows"][0] + st["qkv_rows"][1], sum(st["qkv_rows"])
                L.q, L.k, L.v = L.qkv.rows(0, r1), L.qkv.rows(r1, r2), L.qkv.rows(r2, r3)

    @property
    def streaming(self) -> bool:
        return bool(self._stream)

    def _issue_copy(self, l: int) -> None:
        slot, st = (l - self.streamed_from) & 1, self._stream[l]
        with torch.cuda.stream(self._side):
            if self._freed_valid[slot]:
                self._side.wait_event(self._freed[slot])     # the layer that used this buffer last has been consumed
            self._slots[slot][:st["bytes"]].copy_(st["host"], non_blocking=True)
            self._ready[slot].record(self._side)
        self._slot_layer[slot] = l
        self.stream_copies += 1

    def acquire_layer(self, l: int) -> None:
        """Before the first launch of layer ``l``: its matrices are (being) copied into their buffer; the current stream waits."""
        if l < self.streamed_from or not self._stream:
            return
        slot = (l - self.streamed_from) & 1
        if self._slot_layer[slot] != l:
            self._issue_copy(l)
        torch.cuda.current_stream(self.device).wait_event(self._ready[slot])

    def release_layer(self, l: int, prefetch: Optional[int] = None) -> None:
        """After the last launch of layer ``l``: its buffer may be refilled; ``prefetch`` names the layer to start copying into it."""
        if l < self.streamed_from or not self._stream:
            return
        slot = (l - self.streamed_from) & 1
        self._freed[slot].record(torch.cuda.current_stream(self.device))
        self._freed_valid[slot] = True
        if prefetch is not None and prefetch != l and prefetch >= self.streamed_from and ((prefetch - self.streamed_from) & 1) == slot:
            self._issue_copy(prefetch)

    def prefetch_after(self, order: Sequence[int], i: int) -> Optional[int]:
        """The layer to prefetch when ``order[i]`` is done, for a pass that visits the layers in ``order``: the streamed layer two
        places on (the next one already sits in the other buffer), wrapping to the start of the next pass."""
        s = [l for l in order if l >= self.streamed_from]
        if len(s) <= 2 or order[i] not in s:
            return None
        return s[(s.index(order[i]) + 2) % len(s)]

    def weight_bytes(self) -> int:
        tot = self.lm_head.nbytes
        for L in self.layers:
            for w in (L.q, L.k, L.v, L.o, L.gate, L.up, L.down):
                if w is not None:
                    tot += w.nbytes
        return tot


@dataclass
class StepBuffers:
    """Static device buffers of a decode step for up to ``max_batch`` sequences."""
    tokens: torch.Tensor
    positions: torch.Tensor
    page_table: torch.Tensor
    x: torch.Tensor            # residual stream [B, hidden]
    y1: torch.Tensor           # qkv (+ MLP activation for parallel-residual models)
    attn_out: torch.Tensor     # o_proj input (padded to the covering blocks under TP)
    act: torch.Tensor          # down-proj input
    partial_out: Optional[torch.Tensor]   # row-parallel partial sums awaiting the all-reduce (TP only)
    logits: torch.Tensor
    sampled: torch.Tensor
    temperature: torch.Tensor
    top_k: torch.Tensor
    top_p: torch.Tensor
    min_p: torch.Tensor
    uniform: torch.Tensor
    attn_partial: torch.Tensor
    attn_counters: torch.Tensor
    local_val: Optional[torch.Tensor] = None     # TP: this rank's best logit per sequence
    local_idx: Optional[torch.Tensor] = None     # TP: its global token id
    logits_full: Optional[torch.Tensor] = None   # TP sampling: gathered logits
    act_q: Optional[torch.Tensor] = None         # batch 1: the MLP activation as the int8 block the down-projection launch stages
    # per-sequence logit controls of sampling plans (None on greedy-only engines)
    history: Optional[torch.Tensor] = None       # [B, window] ring of recent token ids (-1: empty)
    repetition: Optional[torch.Tensor] = None    # [B] repetition penalty (1 = off)
    presence: Optional[torch.Tensor] = None      # [B]
    frequency: Optional[torch.Tensor] = None     # [B]
    bias: Optional[torch.Tensor] = None          # [B, vocab] additive row: logit_bias entries, -inf for tokens a grammar forbids
    bias_on: Optional[torch.Tensor] = None       # [B] int32: row b of `bias` is in use


def _is_fast(w: DeviceWeight) -> bool:
    from ..quant.device_layout import FAST_TYPES
    return QType(w.qtype) in FAST_TYPES


# Timing diagnostic only (results are wrong): RLZ_DIAG_SKIP=attn,qkv,oproj leaves those launches out of the decode plan so
# that the marginal cost of a kernel inside the real launch sequence can be read from the step time.
_DIAG_SKIP = set(filter(None, os.environ.get("RLZ_DIAG_SKIP", "").split(",")))


class DecodePlan:
    """The launch sequence of one decode step for a fixed batch size; ``run()`` issues it on
    the current stream (eagerly or under graph capture)."""

    def __init__(self, sm_count: int = 148):
        self.sm_count = sm_count
        self.thunks: List[Callable[[], None]] = []
        self.records: list = []             # one entry per thunk: ("gemv", params) | ("attn", params) | ("embed", args) | ("argmax", args) | None
        self.keep: list = []
        self.kernel_launches = 0
        self.program = None                 # persistent step program, when the plan was compiled into one
        self._side: Optional[torch.cuda.Stream] = None
        self._side_mode = False
        self._ev_fork: Optional[torch.cuda.Event] = None
        self._ev_join: Optional[torch.cuda.Event] = None

    # -- a second stream for work that is independent of the main chain (captured as a parallel graph branch) --
    def fork(self) -> None:
        """Launches added until ``join()`` run on a lower-priority side stream, concurrently with the
        launches added to the main chain after ``join_later()``."""
        def _fork():
            if self._side is None:
                self._side = torch.cuda.Stream(priority=0)
                self._ev_fork, self._ev_join = torch.cuda.Event(), torch.cuda.Event()
            self._ev_fork.record()
            self._side.wait_event(self._ev_fork)
        self.thunks.append(_fork)
        self.records.append(None)
        self._side_mode = True

    def end_fork(self) -> None:
        self._side_mode = False

    def join(self) -> None:
        def _join():
            self._ev_join.record(self._side)
            torch.cuda.current_stream().wait_event(self._ev_join)
        self.thunks.append(_join)
        self.records.append(None)

    def _push(self, fn, record=None) -> None:
        if self._side_mode:
            def on_side(fn=fn):
                with torch.cuda.stream(self._side):
                    fn()
            self.thunks.append(on_side)
            self.records.append(None)
        else:
            self.thunks.append(fn)
            self.records.append(record)

    def add_gemv(self, p, stream=False, tag=""):
        self.keep.append(p)
        if tag and tag in _DIAG_SKIP:
            return
        fn = ops.gemv_stream_launch if stream else ops.gemv_launch
        self._push(lambda p=p, fn=fn: fn(p), None if stream else ("gemv", p))
        self.kernel_launches += 1

    def add_gemv_auto(self, xs, mats, y, batch, ldy, residual=None, ld_res=None, target_ctas=296, ar=None, tag=""):
        """Emit one GEMV launch, or several when the matrices mix int8-fast-path block types with
        generic ones (a launch is homogeneous).  A two-matrix accumulate of mixed kinds becomes two
        launches, the second one accumulating onto the output of the first."""
        fast, generic = [], []
        for m in mats:
            kinds = {_is_fast(w) for w, _ in m.segs}
            if len(kinds) == 2:
                if m.combine != COMBINE_ADD or m.out_off != 0 or len(mats) != 1 or ar is not None:
                    raise ValueError("gated pairs must share a block-type family")
                (w0, x0), (w1, x1) = m.segs
                first = MatOut([(w0, 0)], bias=m.bias, act=ACT_NONE, residual=m.residual)
                self.add_gemv(ops.build_gemv_params([xs[x0]], [first], y, batch, ldy=ldy, residual=residual, ld_res=ld_res, target_ctas=target_ctas))
                second = MatOut([(w1, 0)], bias=m.bias2, act=m.act, residual=True)
                self.add_gemv(ops.build_gemv_params([xs[x1]], [second], y, batch, ldy=ldy, residual=y, ld_res=ldy, target_ctas=target_ctas))
                return
            (fast if kinds == {True} else generic).append(m)
        for group in (fast, generic):
            if group:
                st = group is fast and ops.stream_eligible(group)
                self.add_gemv(ops.build_gemv_params(xs, group, y, batch, ldy=ldy, residual=residual, ld_res=ld_res,
                                                    target_ctas=self.sm_count if st else target_ctas, ar=ar), stream=st, tag=tag)

    def add_attn(self, p):
        self.keep.append(p)
        if "attn" in _DIAG_SKIP:
            return
        self.thunks.append(lambda p=p: ops.attn_decode_launch(p))
        self.records.append(("attn", p))
        self.kernel_launches += 1

    def add(self, fn, launches=1, record=None):
        self.thunks.append(fn)
        self.records.append(record)
        self.kernel_launches += launches

    def compile_persistent(self, device, occ: int, attn_gt: int) -> bool:
        """Fuse the leading run of embedding / GEMV / attention / argmax launches into one persistent
        cooperative kernel (``ops.step_program``).  Returns False, leaving the plan untouched, when the
        run is too short or holds an operation the step kernel does not take."""
        from ..ops.step_program import StepProgramBuilder
        n = 0
        while n < len(self.records) and self.records[n] is not None:
            n += 1
            if self.records[n - 1][0] == "argmax":
                break
        if n < 3:
            return False
        b = StepProgramBuilder(ops.lib(), device, occ, attn_gt, self.sm_count)
        slots = b.grid * 4
        scratch = None
        try:
            for kind, arg in self.records[:n]:
                if kind == "gemv":
                    b.add_gemv(arg)
                elif kind == "attn":
                    q = type(arg).from_buffer_copy(bytes(arg))
                    gx = q.n_kv_heads * -(-(q.n_heads // q.n_kv_heads) // attn_gt)
                    q.splits = max(1, min(32, slots // max(1, gx)))
                    if scratch is None:
                        scratch = (torch.zeros(q.n_heads * q.splits * (q.head_dim + 2), dtype=torch.float32, device=device),
                                   torch.zeros(max(1, q.n_heads), dtype=torch.int32, device=device))
                        self.keep.append(scratch)
                    q.partial, q.counters = scratch[0].data_ptr(), scratch[1].data_ptr()
                    b.add_attn(q)
                elif kind == "embed":
                    b.add_embed(*arg)
                else:
                    b.add_argmax(*arg)
            program = b.finish()
        except ValueError as e:
            log.info("decode plan stays one launch per operation: %s", e)
            return False
        self.program = program
        rest = self.thunks[n:]

        def launch_program(program=program):
            ops.check(program.launch(ops.stream_ptr()), "decode_step")
        self.thunks = [launch_program] + rest
        self.records = [None] * len(self.thunks)
        self.kernel_launches = self.kernel_launches - n + 1
        return True

    def run(self, profiler=None):
        """Issue the launches on the current stream.  With ``profiler`` (``utils.trace.BrickProfiler``) every launch is
        bracketed by events under the name of its kind."""
        if profiler is None:
            for t in self.thunks:
                t()
            return
        for t, rec in zip(self.thunks, self.records):
            with profiler.brick(rec[0] if rec is not None else "other"):
                t()


def emit_head(plan: "DecodePlan", model: GpuModel, buf: StepBuffers, r0: int, batch: int, comm, greedy_only: bool, sm_count: int,
              target_ctas: Optional[int] = None) -> None:
    """Final norm + lm_head + token selection for rows ``r0 .. r0+batch-1`` of the step buffers."""
    cfg = model.cfg
    H = cfg.hidden_dim
    norm_t = NORM_LAYER if cfg.uses_layernorm else NORM_RMS
    for c0 in range(0, batch, 4):
        cb = min(4, batch - c0)
        xin = VecIn(buf.x[r0 + c0:], H, ld=buf.x.stride(0), norm=norm_t, norm_w=model.out_norm_w, norm_b=model.out_norm_b, eps=cfg.eps)
        plan.add_gemv_auto([xin], [MatOut([(model.lm_head, 0)], bias=model.lm_head_b)], buf.logits[r0 + c0:], cb,
                           buf.logits.stride(0),
                           target_ctas=target_ctas or int(os.environ.get("RLZ_GEMV_CTAS", 2 * sm_count if cb <= 1 else sm_count)))
    emit_select(plan, model, buf, r0, batch, comm, greedy_only)


def emit_select(plan: "DecodePlan", model: GpuModel, buf: StepBuffers, r0: int, batch: int, comm, greedy_only: bool) -> None:
    """Token selection from ``buf.logits`` rows ``r0 .. r0+batch-1`` into ``buf.sampled``."""
    V = model.cfg.vocab_size
    tp = model.tp_size > 1
    fused = tp and getattr(comm, "fused", False)
    rows = slice(r0, r0 + batch)

    def controls(logits_rows, v0: int = 0, vn: int = V):
        """History update and per-sequence logit controls ahead of the sampling kernel (sampling plans only); ``v0`` / ``vn``:
        the vocabulary slice that ``logits_rows`` holds."""
        if buf.history is None:
            return 0
        def run():
            ops.history_push(buf.history[rows], buf.tokens[rows], buf.positions[rows], batch)
            ops.logit_controls(logits_rows, buf.history[rows], buf.repetition[rows], buf.presence[rows], buf.frequency[rows],
                               buf.bias[rows, v0:v0 + vn], buf.bias_on[rows], index_offset=v0, vocab=vn)
        plan.add(run, launches=2)
        return 2
    if tp and greedy_only:
        def pick():
            ops.argmax(buf.logits[rows], out=buf.local_idx[rows], out_val=buf.local_val[rows], index_offset=model.vocab_start, vocab=model.vocab_local)
            comm.select_greedy(buf.local_val[rows], buf.local_idx[rows], buf.sampled[rows], batch)
        plan.add(pick, launches=2 if fused else 1)
    elif fused and getattr(comm, "sbuf", None) is not None and os.environ.get("RLZ_SHARDED_SAMPLING", "1") != "0":
        # every rank selects the candidates of its vocabulary slice, the lists are exchanged over peer memory and every rank
        # draws the same token from the merged list: no rank ever holds the whole vocabulary row
        sp_loc = ops.build_sample_params(buf.logits[rows], buf.temperature[rows], buf.top_k[rows], buf.top_p[rows], buf.uniform[rows],
                                         buf.sampled[rows], buf.min_p[rows], vocab=model.vocab_local)
        desc = comm.shard_sample_desc(model.vocab_start)
        plan.keep += [sp_loc, desc]
        controls(buf.logits[rows], model.vocab_start, model.vocab_local)
        plan.add(lambda: comm.sample_sharded(sp_loc, desc), launches=2)
    elif tp:
        sp_full = ops.build_sample_params(buf.logits_full[rows], buf.temperature[rows], buf.top_k[rows], buf.top_p[rows], buf.uniform[rows],
                                          buf.sampled[rows], buf.min_p[rows], vocab=V)
        plan.keep.append(sp_full)

        def pick_sampled():
            buf.logits_full[rows].copy_(comm.gather_logits(buf.logits[rows, :model.vocab_local], V))
        plan.add(pick_sampled, launches=0)
        controls(buf.logits_full[rows])
        plan.add(lambda: ops.sample_launch(sp_full), launches=1)
    elif greedy_only:
        plan.add(lambda: ops.argmax(buf.logits[rows], out=buf.sampled[rows], vocab=V),
                 record=("argmax", (buf.logits[rows], V, buf.sampled[rows])) if batch == 1 else None)
    else:
        sp = ops.build_sample_params(buf.logits[rows], buf.temperature[rows], buf.top_k[rows], buf.top_p[rows], buf.uniform[rows],
                                     buf.sampled[rows], buf.min_p[rows], vocab=V)
        plan.keep.append(sp)
        controls(buf.logits[rows])
        plan.add(lambda: ops.sample_launch(sp))


def build_decode_plan(model: GpuModel, buf: StepBuffers, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: int, splits: int,
                      comm=None, greedy_only: bool = False, sm_count: int = 148, layer_subset: Optional[Sequence[int]] = None,
                      persistent: bool = False) -> DecodePlan:
    """Create the launch plan for ``batch`` sequences (rows 0..batch-1 of the step buffers).
    ``layer_subset`` restricts the pass to those layers (the layer-skipping draft of self-speculative decoding).

    ``k_cache`` / ``v_cache`` are ``[layers, pages, kv_heads, 16, head_dim]`` bf16.  ``comm`` is the
    tensor-parallel communicator (``None`` on one GPU); it provides ``all_reduce_sum_(tensor)``.
    """
    cfg = model.cfg
    plan = DecodePlan(sm_count)
    H, hd = cfg.hidden_dim, cfg.head_dim
    qd, kvd, I = model.q_dim, model.kv_dim, model.inter
    norm_t = NORM_LAYER if cfg.uses_layernorm else NORM_RMS
    tp = model.tp_size > 1
    target = int(os.environ.get("RLZ_GEMV_CTAS", 2 * sm_count if batch <= 1 else sm_count))   # register-path kernel: 2 CTAs/SM at batch 1
    # persistent step kernel (batch 1, one GPU): the whole step is one cooperative launch; its grid is 2 CTAs per SM for
    # multi-head attention and 1 CTA per SM (twice the registers) when an attention job carries several query heads
    p_occ = p_gt = 0
    if persistent and batch == 1 and model.tp_size == 1:
        G = model.heads // max(1, model.kv_heads)
        p_gt = 1 if G == 1 else 2 if G == 2 else 0 if G == 8 else 4
        p_occ = int(os.environ.get("RLZ_PERSIST_OCC", 2 if p_gt == 1 else 1)) if p_gt else 0
        if p_occ == 2 and p_gt != 1:
            p_occ = 1
        if p_occ:
            target = p_occ * sm_count
    chunks = [(c, min(4, batch - c)) for c in range(0, batch, 4)]       # GEMV kernels take <= 4 rows at a time
    # batch 1, one GPU: the launch that produces the MLP activation also writes it as the int8 block that the down-projection
    # launch stages, so all of that launch's CTAs copy 1.9 bytes per value instead of reading 4 and quantising
    def handoff(L) -> bool:
        # (tensor parallel: only when this rank's activation slice starts on a block boundary of the down projection's shard)
        return (batch == 1 and (not tp or L.down_in_off == 0) and buf.act_q is not None and os.environ.get("RLZ_ACT_HANDOFF", "1") != "0" and _is_fast(L.down)
                and _is_fast(L.up) and (L.gate is None or _is_fast(L.gate)) and L.down.k % 128 == 0 and L.up.n == L.down.k
                and buf.act_q.numel() >= ops.act_block_bytes(L.down.k))
    overlap_up = cfg.parallel_residual and len(chunks) == 1 and os.environ.get("RLZ_OVERLAP_UP", "0") == "1"   # measured slower than the single chain; opt-in
    qkv_w = qd + 2 * kvd
    ld1 = buf.y1.stride(0)

    plan.add(lambda: ops.embed(model.embed_table, model.embed_qtype, model.embed_row_bytes, H, cfg.vocab_size, buf.tokens[:batch], buf.x,
                               model.pos_table, buf.positions),
             record=("embed", (model.embed_table, model.embed_qtype, model.embed_row_bytes, H, cfg.vocab_size, buf.tokens[:batch], buf.x,
                               model.pos_table, buf.positions)) if batch == 1 else None)

    fused = tp and getattr(comm, "fused", False)
    site = [0]
    if fused:
        plan.add(comm.begin_step, launches=comm.step_launches())

    def reduce_into_x(partial_rows):
        """Baseline TP: x += all_reduce(partial) as a library collective plus one residual-add launch."""
        comm.all_reduce_sum_(partial_rows)
        ops.elementwise(partial_rows, residual=buf.x[:batch], out=buf.x[:batch])

    def row_parallel(xs_of, mat_of):
        """Emit the row-parallel GEMV(s) of a layer: x += W_shard . inputs (+ bias on rank 0), all-reduced
        across ranks.  One GPU: a plain fused-residual GEMV.  Fused TP: the all-reduce happens inside the
        kernel.  Baseline TP: partial sums, NCCL all-reduce, residual-add kernel."""
        mixed = len({_is_fast(w) for w, _ in mat_of(True).segs}) == 2     # block-type families that cannot share a launch
        use_ar = fused and not mixed
        for c0, cb in chunks:
            mat = mat_of(not tp or use_ar)
            if not tp or use_ar:
                ar = None
                if use_ar:
                    ar = comm.ar_desc(site[0])
                    site[0] += 1
                plan.add_gemv_auto(xs_of(c0), [mat], buf.x[c0:], cb, buf.x.stride(0), residual=buf.x[c0:], ld_res=buf.x.stride(0),
                                   target_ctas=target, ar=ar, tag="oproj")
            else:
                plan.add_gemv_auto(xs_of(c0), [mat], buf.partial_out[c0:], cb, buf.partial_out.stride(0), target_ctas=target)
        if tp and not use_ar:
            plan.add(lambda: reduce_into_x(buf.partial_out[:batch]), launches=1)

    order = [l for l in range(len(model.layers)) if layer_subset is None or l in layer_subset]
    for l, L in enumerate(model.layers):
        if layer_subset is not None and l not in layer_subset:
            continue
        kc, vc = k_cache[l], v_cache[l]
        if model.streaming and l >= model.streamed_from:     # streamed layer: wait for its matrices (stream operations, no launch)
            plan.add(lambda l=l: model.acquire_layer(l), launches=0)
        for c0, cb in chunks:
            x = buf.x[c0:]
            xin = VecIn(x, H, ld=buf.x.stride(0), norm=norm_t, norm_w=L.attn_norm_w, norm_b=L.attn_norm_b, eps=cfg.eps)
            mats = [MatOut([(L.q, 0)], out_off=0, bias=L.q_b), MatOut([(L.k, 0)], out_off=qd, bias=L.k_b),
                    MatOut([(L.v, 0)], out_off=qd + kvd, bias=L.v_b)]
            if cfg.parallel_residual:
                up_mat = MatOut([(L.up, 0)], out_off=model.act_col0 + L.down_in_off, bias=L.up_b,
                                act=ACT_GELU if cfg.constraints.activation == "gelu" else ops.ACT_SILU)
                if handoff(L):
                    up_mat.q_out, up_mat.q_out_k, up_mat.q_out_col0 = buf.act_q, L.down.k, 0
                if overlap_up:
                    # the MLP up-projection does not depend on attention: it streams its weights on a side
                    # stream while the main chain runs QKV -> attention (whose latency it hides)
                    plan.fork()
                    plan.add_gemv_auto([xin], [up_mat], buf.y1[c0:], cb, ld1, target_ctas=target)
                    plan.end_fork()
                else:
                    mats.append(up_mat)
            plan.add_gemv_auto([xin], mats, buf.y1[c0:], cb, ld1, target_ctas=target, tag="qkv")
        plan.add_attn(ops.build_attn_decode_params(
            buf.y1, buf.attn_out[:, L.o_in_off:], kc, vc, buf.positions, buf.page_table, buf.attn_partial, buf.attn_counters,
            model.heads, model.kv_heads, hd, splits, batch, cfg.rope_dim if cfg.uses_rope else 0, cfg.rope_type, cfg.rope_theta,
            0, qd, qd + kvd, L.q_norm_w, L.k_norm_w, cfg.eps, ld_qkv=ld1, ld_out=buf.attn_out.stride(0),
            window=cfg.sliding_window or 0, rope_table=model.rope_table if cfg.uses_rope else None))
        if cfg.parallel_residual and overlap_up:
            plan.join()
        if cfg.parallel_residual:
            row_parallel(lambda c0: [VecIn(buf.attn_out[c0:], L.o.k, ld=buf.attn_out.stride(0)),
                                     VecIn(buf.y1[c0:, model.act_col0:], L.down.k, ld=ld1, pre=buf.act_q if handoff(L) else None)],
                         lambda res: MatOut([(L.o, 0), (L.down, 1)], bias=L.o_b, bias2=L.down_b, combine=COMBINE_ADD, residual=res))
        else:
            row_parallel(lambda c0: [VecIn(buf.attn_out[c0:], L.o.k, ld=buf.attn_out.stride(0))],
                         lambda res: MatOut([(L.o, 0)], bias=L.o_b, residual=res))
            for c0, cb in chunks:
                xin = VecIn(buf.x[c0:], H, ld=buf.x.stride(0), norm=norm_t, norm_w=L.ffn_norm_w, norm_b=L.ffn_norm_b, eps=cfg.eps)
                if cfg.gated_ffn:
                    comb = COMBINE_SILU_MUL if cfg.constraints.activation == "silu" else COMBINE_GELU_MUL
                    mat = MatOut([(L.gate, 0), (L.up, 0)], combine=comb, bias2=L.up_b)
                else:
                    mat = MatOut([(L.up, 0)], bias=L.up_b, act=ACT_GELU if cfg.constraints.activation == "gelu" else ops.ACT_SILU)
                if handoff(L):
                    mat.q_out, mat.q_out_k, mat.q_out_col0 = buf.act_q, L.down.k, 0
                plan.add_gemv_auto([xin], [mat], buf.act[c0:, L.down_in_off:], cb, buf.act.stride(0), target_ctas=target)
            row_parallel(lambda c0: [VecIn(buf.act[c0:], L.down.k, ld=buf.act.stride(0), pre=buf.act_q if handoff(L) else None)],
                         lambda res: MatOut([(L.down, 0)], bias=L.down_b, residual=res))
        if model.streaming and l >= model.streamed_from:
            plan.add(lambda l=l, nxt=model.prefetch_after(order, order.index(l)): model.release_layer(l, nxt), launches=0)

    emit_head(plan, model, buf, 0, batch, comm, greedy_only, sm_count, target_ctas=target if p_occ else None)
    plan.ar_sites = site[0]
    if p_occ:
        plan.compile_persistent(buf.x.device, p_occ, p_gt)
    return plan
