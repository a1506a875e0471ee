"""Token-batch forward pass on the tensor-core GEMM path: prompt prefill (one sequence, many
tokens) and decode steps of batches too large for the GEMV kernels (many sequences, one token).

Per layer and token batch of T rows:
``norm -> bf16`` -> GEMM Q/K/V (+bias) -> [QK-norm] -> RoPE -> paged KV append ->
attention over the paged cache (the decode kernel with one "sequence" per token row) ->
``bf16`` -> GEMM o_proj (+residual) -> ``norm -> bf16`` -> GEMM gate/up -> SwiGLU/GELU ->
GEMM down (+residual).  Everything is a static launch sequence over preallocated buffers, so a
whole pass can be captured in a CUDA graph per token-count bucket.

Replaces the reference's ``prefill_all_layers_gpu`` / ``transformer_layer_batched`` chain
(src/cuda/executor/layers/prefill.rs:31-490, src/cuda/executor/layers/transformer_layer_batched.rs:24-143),
whose GEMMs are cuBLAS calls and whose attention is strided-batched SGEMM + a softmax kernel.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from .. import ops
from ..ops import ACT_GELU, ACT_NONE, ACT_SILU, NORM_LAYER, NORM_RMS, gemm as G
from .decoder import GpuModel


def gemm_capable(model: GpuModel) -> bool:
    """True when every projection of the model can run on the tensor-core GEMM kernel."""
    ws = [model.lm_head]
    for L in model.layers:
        ws += [w for w in (L.q, L.k, L.v, L.o, L.gate, L.up, L.down) if w is not None]
    return all(G.gemm_eligible(w) for w in ws)


class BatchedForward:
    def __init__(self, model: GpuModel, max_tokens: int, k_cache: torch.Tensor, v_cache: torch.Tensor, max_pages: int, comm=None,
                 sm_count: int = 148):
        self.model, self.comm, self.sm_count = model, comm, sm_count
        self.T = max_tokens
        cfg = model.cfg
        dev = model.device
        H, qd, kvd, I = cfg.hidden_dim, model.q_dim, model.kv_dim, model.inter
        self.qkv_w = qd + 2 * kvd
        o_k = max(L.o.k for L in model.layers)
        d_k = max(L.down.k for L in model.layers)
        T = max_tokens
        z = lambda *s, dt=torch.float32: torch.zeros(*s, device=dev, dtype=dt)
        self.tokens, self.positions, self.page_rows = z(T, dt=torch.int32), z(T, dt=torch.int32), z(T, dt=torch.int32)
        self.x = z(T, H)
        self.xb = z(T, H, dt=torch.bfloat16)
        self.qkv = z(T, self.qkv_w)
        self.attn = z(T, o_k)                       # zero padding around this rank's slice under TP
        self.attn_b = z(T, o_k, dt=torch.bfloat16)
        self.gate, self.up = z(T, I), (z(T, I) if cfg.gated_ffn else None)
        self.act_b = z(T, d_k, dt=torch.bfloat16)   # down-proj input (padded under TP)
        self.partial = z(T, H) if model.tp_size > 1 else None
        self.k_cache, self.v_cache = k_cache, v_cache
        self.max_pages = max_pages
        self.splits = 1
        self.attn_partial, self.attn_counters = ops.attn_decode_scratch(T, model.heads, self.splits, cfg.head_dim, dev)
        self.launches_per_pass = 0
        self.flash_ok = ops.attn_prefill_supported(cfg.head_dim) and self.attn.stride(0) % 4 == 0
        self.flash_min_tokens = 16
        # tensor parallel, fused mode: row-parallel GEMMs of up to ll_tokens rows push their partial tiles into the peers'
        # inboxes from the epilogue (one-shot all-reduce, latency-optimal); longer chunks use NCCL (bandwidth-optimal)
        self.ll_tokens = 0
        # tensor parallel, fused mode (default): two-shot all-reduce.  The row-parallel GEMM stores each token row's partial
        # result only into the inbox of the rank that owns the row; the owner sums the partials onto its fp32 residual row,
        # applies the norm that follows and sends the bf16 row to every rank's operand buffer, which the next GEMM reads from
        # local memory.  Between layers the residual stream is therefore kept per owner; the last site of a pass sends the fp32
        # rows to every rank instead.  x and xb live in the communicator's symmetric memory.
        self.two_shot = (model.tp_size > 1 and getattr(comm, "fused", False) and H % 4 == 0 and H <= 8192
                         and os.environ.get("RLZ_TWO_SHOT", "1") != "0")
        if self.two_shot:
            comm.allocate_two_shot(cfg.num_layers * (1 if cfg.parallel_residual else 2), H, max_tokens)
            self.x, self.xb = comm.ts_x[:, :H], comm.ts_xb[:, :H]
        elif model.tp_size > 1 and getattr(comm, "fused", False):
            # measured: at 64 rows the one-shot push loses to NCCL at every world size (2 GPUs 0.76x, 4 GPUs 0.98x,
            # 8 GPUs 0.67x of the NCCL step rate); it is kept for the short batches where latency decides
            self.ll_tokens = min(max_tokens, int(os.environ.get("RLZ_LL_TOKENS", max(8, 64 // model.tp_size))))
            comm.allocate_gemm(2 * cfg.num_layers, H, self.ll_tokens)
        self._site = 0
        # prompt chunks of one sequence: the page-table row and the chunk position are read from static device buffers, so the
        # launch sequence of a chunk of T tokens is the same for every sequence and position and is replayed from a CUDA graph
        self.pt_row = z(max_pages, dt=torch.int32)
        self._chunk_graphs: dict = {}
        self._chunk_seen: dict = {}
        self.chunk_graphs = os.environ.get("RLZ_PREFILL_GRAPHS", "1") != "0"

    def forward_chunk(self, T: int, page_table_row: torch.Tensor, pos0: int) -> torch.Tensor:
        """Rows 0..T-1 are positions ``pos0 .. pos0+T-1`` of the sequence whose page-table row is given (``tokens`` /
        ``positions`` / ``page_rows`` must be set).  The first pass of a given T runs launch by launch; full-size chunks (and
        any T seen twice) are then captured and replayed as one graph, which removes the host's launch work (some hundred
        launches per pass) from the time to first token - under tensor parallelism the pass is otherwise host-bound."""
        self.pt_row.copy_(page_table_row, non_blocking=True)
        g = self._chunk_graphs.get(T)
        if g is not None:
            g.replay()
            return self.x[:T]
        x = self.forward(T, self.pt_row, shared_table=True, pos0=pos0, pos0_dev=self.positions)
        seen = self._chunk_seen[T] = self._chunk_seen.get(T, 0) + 1
        if self.chunk_graphs and not self.model.streaming and len(self._chunk_graphs) < 16 and (T == self.T or seen >= 2):
            torch.cuda.synchronize(self.model.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.forward(T, self.pt_row, shared_table=True, pos0=pos0, pos0_dev=self.positions)
            self._chunk_graphs[T] = graph
        return x

    # -- helpers ---------------------------------------------------------------------------
    def _gemm(self, w, x_b, y, T, bias=None, act=ACT_NONE, residual_inplace=False, y_col=0):
        """y[:, y_col:y_col+n] (+)= x_b W^T.  ``residual_inplace``: y already holds the residual."""
        yv = y[:, y_col:]
        if residual_inplace:
            sk = G.choose_splitk(w.n, w.k, T, self.sm_count)
            if sk > 1:
                G.gemm_launch(G.build_gemm_params(w, x_b, yv, T, bias=bias, splitk=sk, ldy=y.stride(0)))
            else:
                G.gemm_launch(G.build_gemm_params(w, x_b, yv, T, bias=bias, residual=yv, ldy=y.stride(0), ld_res=y.stride(0)))
        else:
            sk = G.choose_splitk(w.n, w.k, T, self.sm_count) if act == ACT_NONE else 1
            if sk > 1:                                      # few tokens: split K for occupancy, partial products add into zeros
                y[:T, y_col:y_col + w.n].zero_()
                self.launches_per_pass += 1
            G.gemm_launch(G.build_gemm_params(w, x_b, yv, T, bias=bias, act=act, splitk=sk, ldy=y.stride(0)))
        self.launches_per_pass += 1

    def _gemm_to_operand(self, w, x_b, dst_b, T, bias, act, mul=None) -> bool:
        """dst_b[:T, :n] = bf16(act(x_b W^T + bias) [* mul]) written by the GEMM epilogue (no fp32 round trip, no
        separate activation launch).  Returns False when K would be split for occupancy (the caller then takes the
        fp32 path followed by the activation kernel)."""
        if G.choose_splitk(w.n, w.k, T, self.sm_count) != 1:
            return False
        G.gemm_launch(G.build_gemm_params(w, x_b, dst_b, T, bias=bias, act=act, residual=mul, ldy=dst_b.stride(0),
                                          ld_res=mul.stride(0) if mul is not None else None, res_mul=mul is not None))
        self.launches_per_pass += 1
        return True

    def _two_shot(self, w, x_b, T, bias, local_partial, next_norm, final: bool) -> None:
        """x += sum over ranks of (W_shard . x_b + bias [+ local_partial]) by the two-shot all-reduce; then either the bf16
        operand of the following GEMMs (``next_norm`` = (kind, weight, bias) of the norm that follows) or, at the last site
        of a pass (``final``), the fp32 residual rows arrive on every rank."""
        sk = G.choose_splitk(w.n, w.k, T, self.sm_count)
        p = G.build_gemm_params(w, x_b, self.partial, T, bias=bias, residual=local_partial, splitk=sk, ldy=self.partial.stride(0),
                                ld_res=self.partial.stride(0) if local_partial is not None else None)
        self.comm.two_shot_fill(p, self._site, T)
        G.gemm_launch(p)
        kind, nw, nb = next_norm if next_norm is not None else (ops.NORM_NONE, None, None)
        self.comm.two_shot_reduce(p, self._site, T, kind, nw, nb, self.model.cfg.eps, to_xb=not final, push_x=final)
        self._site += 1
        self.launches_per_pass += 2

    def _row_parallel(self, w, x_b, T, bias):
        """x += W_shard . x_b (+ bias), summed over tensor-parallel ranks."""
        if self.model.tp_size == 1:
            self._gemm(w, x_b, self.x, T, bias=bias, residual_inplace=True)
            return
        if 0 < T <= self.ll_tokens:
            p = G.build_gemm_params(w, x_b, self.partial, T, bias=bias, ldy=self.partial.stride(0))
            self.comm.gemm_ar_fill(p, self._site)
            G.gemm_launch(p)
            self.comm.ll_reduce(self._site, self.x, T, w.n, w.k)
            self._site += 1
            self.launches_per_pass += 2
            return
        self._gemm(w, x_b, self.partial, T, bias=bias)
        self.comm.all_reduce_sum_(self.partial[:T])
        ops.elementwise(self.partial[:T], residual=self.x[:T], out=self.x[:T])
        self.launches_per_pass += 1

    # -- the pass ------------------------------------------------------------------------------
    def forward(self, T: int, page_table: torch.Tensor, shared_table: bool, pos0: Optional[int] = None,
                pos0_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run all layers for rows 0..T-1 (``tokens`` / ``positions`` / ``page_rows`` must be set).
        ``page_table``: ``[max_pages]`` shared by all rows (prefill) or ``[T, max_pages]``.
        ``pos0``: rows are the consecutive positions ``pos0 .. pos0+T-1`` of one sequence (a prompt chunk);
        attention then runs on the tensor-core flash kernel instead of one decode-kernel row per token.
        Returns the residual stream ``x[:T]`` (the caller applies the final norm + lm_head)."""
        m, cfg = self.model, self.model.cfg
        H, qd, kvd, hd = cfg.hidden_dim, m.q_dim, m.kv_dim, cfg.head_dim
        norm_t = NORM_LAYER if cfg.uses_layernorm else NORM_RMS
        act_code = ACT_GELU if cfg.constraints.activation == "gelu" else ACT_SILU
        self.launches_per_pass = 0
        if self.model.tp_size > 1 and getattr(self.comm, "fused", False):
            self._site = 0
            self.comm.begin_step()                         # one epoch per pass tags this pass's peer stores (GEMM pushes, candidate exchange)
            self.launches_per_pass += 1
        x, xb, qkv = self.x[:T], self.xb[:T], self.qkv[:T]
        ops.embed(m.embed_table, m.embed_qtype, m.embed_row_bytes, H, cfg.vocab_size, self.tokens[:T], self.x, m.pos_table, self.positions)
        self.launches_per_pass += 1
        ts = self.two_shot
        order = list(range(len(m.layers)))
        for l, L in enumerate(m.layers):
            m.acquire_layer(l)                                 # streamed layers: wait for the copy into their buffer (no-op otherwise)
            nxt = m.layers[l + 1] if l + 1 < len(m.layers) else None
            next_attn_norm = (norm_t, nxt.attn_norm_w, nxt.attn_norm_b) if nxt is not None else None
            if not ts or l == 0:                               # two-shot: the previous layer's reduce wrote this layer's operand
                ops.norm_bf16(x, xb, L.attn_norm_w, L.attn_norm_b, norm_t, cfg.eps)
            if L.qkv is not None:                              # one GEMM over the fused rows: fuller waves, no split-K zero fill
                self._gemm(L.qkv, xb, self.qkv, T, bias=L.qkv_b, y_col=0)
            else:
                self._gemm(L.q, xb, self.qkv, T, bias=L.q_b, y_col=0)
                self._gemm(L.k, xb, self.qkv, T, bias=L.k_b, y_col=qd)
                self._gemm(L.v, xb, self.qkv, T, bias=L.v_b, y_col=qd + kvd)
            up_fused = False
            if cfg.parallel_residual:                          # GELU(fc1) goes straight into the bf16 operand of fc2 when K is not split
                up_fused = self._gemm_to_operand(L.up, xb, self.act_b[:, L.down_in_off:], T, L.up_b, act_code)
                if not up_fused:
                    self._gemm(L.up, xb, self.gate, T, bias=L.up_b)    # activation applied when the bf16 operand is produced
            if L.q_norm_w is not None:
                ops.head_rmsnorm_(qkv, L.q_norm_w, m.heads, hd, cfg.eps)
                ops.head_rmsnorm_(qkv[:, qd:], L.k_norm_w, m.kv_heads, hd, cfg.eps)
                self.launches_per_pass += 2
            if cfg.uses_rope:                                  # the k heads follow the q heads in a row: one launch rotates both
                ops.rope_(qkv, self.positions[:T], m.heads + m.kv_heads, hd, cfg.rope_dim, cfg.rope_type, cfg.rope_theta, table=m.rope_table)
                self.launches_per_pass += 1
            ops.kv_append(qkv[:, qd:], qkv[:, qd + kvd:], self.k_cache[l], self.v_cache[l], self.positions[:T], self.page_rows[:T], m.kv_heads, hd)
            if pos0 is not None and shared_table and T >= self.flash_min_tokens and self.flash_ok and (L.o_in_off * 2) % 16 == 0:
                ops.attn_prefill(self.qkv, self.attn_b[:, L.o_in_off:], self.k_cache[l], self.v_cache[l], page_table, T, pos0, m.heads, m.kv_heads, hd,
                                 q_off=0, window=cfg.sliding_window or 0, pos0_dev=pos0_dev)       # bf16 result, read directly by the o_proj GEMM
                self.launches_per_pass += 3
            else:
                ops.attn_decode_launch(ops.build_attn_decode_params(
                    self.qkv, self.attn[:, L.o_in_off:], self.k_cache[l], self.v_cache[l], self.positions, page_table, self.attn_partial,
                    self.attn_counters, m.heads, m.kv_heads, hd, self.splits, T, 0, cfg.rope_type, cfg.rope_theta, 0, qd, qd + kvd,
                    None, None, cfg.eps, ld_qkv=self.qkv.stride(0), ld_out=self.attn.stride(0), shared_table=shared_table, no_append=True,
                    window=cfg.sliding_window or 0))
                ops.to_bf16(self.attn[:T], self.attn_b[:T])
                self.launches_per_pass += 4
            if ts and cfg.parallel_residual:
                self._gemm(L.o, self.attn_b[:T, : L.o.k], self.partial, T, bias=L.o_b)      # stays local: the down projection adds it before the push
            elif ts:
                self._two_shot(L.o, self.attn_b[:T, : L.o.k], T, L.o_b, None, (norm_t, L.ffn_norm_w, L.ffn_norm_b), final=False)
            else:
                self._row_parallel(L.o, self.attn_b[:T, : L.o.k], T, L.o_b)
            act_dst = self.act_b[:, L.down_in_off:]
            if cfg.parallel_residual:
                if not up_fused:
                    ops.swiglu_bf16(self.gate[:T], None, self.act_b[:T, L.down_in_off:], act_code)
                    self.launches_per_pass += 1
                if ts:
                    self._two_shot(L.down, self.act_b[:T, : L.down.k], T, L.down_b, self.partial, next_attn_norm, final=nxt is None)
                else:
                    self._row_parallel(L.down, self.act_b[:T, : L.down.k], T, L.down_b)
            else:
                if not ts:
                    ops.norm_bf16(x, xb, L.ffn_norm_w, L.ffn_norm_b, norm_t, cfg.eps)
                    self.launches_per_pass += 1
                if cfg.gated_ffn:
                    # act(gate) in fp32 from the first GEMM's epilogue; the second multiplies it in and writes the bf16 operand
                    fused = G.choose_splitk(L.up.n, L.up.k, T, self.sm_count) == 1 and G.choose_splitk(L.gate.n, L.gate.k, T, self.sm_count) == 1
                    if fused:
                        self._gemm(L.gate, xb, self.gate, T, act=act_code)
                        self._gemm_to_operand(L.up, xb, act_dst, T, L.up_b, ACT_NONE, mul=self.gate)
                    else:
                        self._gemm(L.gate, xb, self.gate, T)
                        self._gemm(L.up, xb, self.up, T, bias=L.up_b)
                        ops.swiglu_bf16(self.gate[:T], self.up[:T], self.act_b[:T, L.down_in_off:], act_code)
                        self.launches_per_pass += 1
                elif not self._gemm_to_operand(L.up, xb, act_dst, T, L.up_b, act_code):
                    self._gemm(L.up, xb, self.gate, T, bias=L.up_b)
                    ops.swiglu_bf16(self.gate[:T], None, self.act_b[:T, L.down_in_off:], act_code)
                    self.launches_per_pass += 1
                if ts:
                    self._two_shot(L.down, self.act_b[:T, : L.down.k], T, L.down_b, None, next_attn_norm, final=nxt is None)
                else:
                    self._row_parallel(L.down, self.act_b[:T, : L.down.k], T, L.down_b)
            m.release_layer(l, m.prefetch_after(order, l) if m.streaming else None)
        return x
