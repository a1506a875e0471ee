"""Builder and launcher of the persistent decode-step kernel (``csrc/kernels/decode_step.cu``).

A step program is a list of operations - embedding lookup, fused GEMVs, attention, argmax - whose
parameter blocks are packed into one device buffer.  One cooperative launch walks the list with a
grid-wide barrier between operations, instead of one kernel launch per operation.

Counterpart of the reference's graph-captured decode step
(src/cuda/executor/layers/graphed_capture.rs:16-364): the same "replay the whole step with one
submission" idea, carried one level further - one kernel, not one graph of a hundred kernels.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch

from . import _signatures as S

STEP_EMBED, STEP_GEMV, STEP_ATTN, STEP_ARGMAX = 0, 1, 2, 3
STATUS_BARRIER_TIMEOUT = 4001


class StepProgramBuilder:
    """Collects operations; ``finish()`` uploads them and returns a launchable :class:`StepProgram`."""

    def __init__(self, lib, device, occ: int, attn_gt: int, sm_count: int):
        self.lib, self.device, self.occ, self.attn_gt, self.sm_count = lib, device, int(occ), int(attn_gt), int(sm_count)
        self.ops: List[Tuple[int, int, bytes]] = []
        self.smem = 1024
        self.keep: list = []

    @property
    def grid(self) -> int:
        return self.occ * self.sm_count

    def add_embed(self, table, qtype: int, row_bytes: int, hidden: int, vocab: int, tokens, out, pos_table=None, positions=None) -> None:
        e = S.StepEmbed()
        e.table, e.tokens, e.out = table.data_ptr(), tokens.data_ptr(), out.data_ptr()
        e.pos_table = pos_table.data_ptr() if pos_table is not None else None
        e.positions = positions.data_ptr() if positions is not None else None
        e.row_bytes, e.qtype, e.hidden, e.vocab = int(row_bytes), int(qtype), int(hidden), int(vocab)
        self.keep += [table, tokens, out, pos_table, positions]
        self.ops.append((STEP_EMBED, 0, bytes(e)))
        self.smem = max(self.smem, 256 * 4)

    def add_gemv(self, p: S.GemvParams) -> None:
        if p.batch != 1 or p.ar.enabled:
            raise ValueError("step programs take batch-1 GEMVs without a fused all-reduce")
        q = S.GemvParams.from_buffer_copy(bytes(p))
        grid = ctypes.c_int(0)
        rc = self.lib.rlz_gemv_prepare(ctypes.byref(q), ctypes.byref(grid))
        if rc != 0:
            raise ValueError(f"GEMV description rejected ({rc})")
        if q.any_generic:
            raise ValueError("step programs take int8-fast-path block types only")
        self.smem = max(self.smem, int(self.lib.rlz_gemv_smem_bytes(ctypes.byref(q))))
        self.keep.append(p)
        self.ops.append((STEP_GEMV, grid.value, bytes(q)))

    def add_attn(self, p: S.AttnDecodeParams) -> None:
        if p.kv_q8 or p.batch != 1:
            raise ValueError("step programs take batch-1 attention over a bf16 cache")
        g = p.n_heads // p.n_kv_heads
        hgroups = -(-g // self.attn_gt)
        jobs = p.n_kv_heads * hgroups * p.splits * p.batch
        sub = int(self.lib.rlz_decode_step_attn_smem(self.attn_gt))
        if sub <= 0:
            raise ValueError("unsupported attention head grouping")
        self.smem = max(self.smem, 4 * sub)
        self.keep.append(p)
        self.ops.append((STEP_ATTN, jobs, bytes(p)))

    def add_argmax(self, logits, vocab: int, out, out_val=None, index_offset: int = 0) -> None:
        a = S.StepArgmax()
        a.logits, a.out, a.out_val = logits.data_ptr(), out.data_ptr(), (out_val.data_ptr() if out_val is not None else None)
        a.vocab, a.index_offset = int(vocab), int(index_offset)
        self.keep += [logits, out, out_val]
        self.ops.append((STEP_ARGMAX, 0, bytes(a)))
        self.smem = max(self.smem, 80 * 4)

    def finish(self, spin_limit: int = 4_000_000) -> "StepProgram":
        if not self.ops:
            raise ValueError("empty step program")
        if any(kind == STEP_ARGMAX for kind, _, _ in self.ops[:-1]):
            raise ValueError("argmax must be the last operation")
        head = ctypes.sizeof(S.StepOp) * len(self.ops)
        off = (head + 15) & ~15
        blob = bytearray(off)
        table = (S.StepOp * len(self.ops))()
        for i, (kind, grid, payload) in enumerate(self.ops):
            table[i].kind, table[i].grid, table[i].params = kind, grid, off
            blob += payload
            blob += bytes((-len(payload)) % 16)
            off = len(blob)
        blob[:head] = bytes(table)
        dev_blob = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.device)
        return StepProgram(self.lib, dev_blob, len(self.ops), self.occ, self.attn_gt, self.smem, spin_limit, self.keep, self.device)


class StepProgram:
    """A launchable step program.  ``launch()`` is asynchronous on the current stream; ``check()`` reads the status word."""

    def __init__(self, lib, blob: torch.Tensor, nops: int, occ: int, attn_gt: int, smem: int, spin_limit: int, keep, device):
        self.lib, self.blob, self.nops, self.smem, self.keep = lib, blob, nops, int(smem), keep
        self.sync = torch.zeros(128, dtype=torch.int32, device=device)     # barrier and argmax words, one 128-byte line each
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        p = S.StepProgram()
        p.blob, p.sync, p.status = blob.data_ptr(), self.sync.data_ptr(), self.status.data_ptr()
        p.spin_limit, p.nops, p.occ, p.attn_gt = int(spin_limit), int(nops), int(occ), int(attn_gt)
        p.skip = int(os.environ.get("RLZ_STEP_SKIP", "0"))        # diagnostics only: leaves out parts of the work
        self.params = p

    def launch(self, stream_ptr: int) -> int:
        return int(self.lib.rlz_decode_step(ctypes.byref(self.params), self.smem, stream_ptr))

    def check(self) -> None:
        """Raise if a barrier wait ran out in an earlier launch; the program is reset so that it can run again."""
        st = int(self.status.item())
        if st != 0:
            self.status.zero_()
            self.sync.zero_()
            raise RuntimeError(f"persistent decode step failed on the device (status {st})")
