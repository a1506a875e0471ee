"""Tensor-parallel communication for the decode engine, one process per GPU.

Two interchangeable communicators:

* ``NcclTpComm`` – the baseline: ``torch.distributed`` (NCCL) all-reduce of the row-parallel
  partial sums followed by a residual-add kernel, NCCL all-gather of argmax candidates / logits.
* ``FusedTpComm`` – the product: row-parallel GEMV kernels all-reduce their own outputs over
  peer memory (each CTA stores its rows into every rank's inbox, publishes an epoch flag, waits
  bounded for the peers and sums in rank order, fused with the residual add; values travel as
  epoch-tagged 8-byte stores, so there are no fences and no separate flags), and the greedy
  token is agreed on by a one-CTA candidate exchange.  No extra launches per all-reduce and no
  library collective on the decode path; buffers are CUDA-IPC-mapped symmetric memory.

The reference has no real communicator (single-process mock,
src/parallel/mod_all_reduce_communicator.rs:2-110).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _signatures as S


class _RawDeviceMemory:
    """CUDA array interface over a raw device address (memory owned by a SymmetricBuffer)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _device_view(ptr: int, nbytes: int, device) -> torch.Tensor:
    """uint8 tensor over ``nbytes`` of device memory at ``ptr`` (no copy, no ownership)."""
    return torch.as_tensor(_RawDeviceMemory(ptr, nbytes), device=device)


class SymmetricBuffer:
    """A zero-initialised device buffer of ``nbytes`` on every rank, mapped into every other rank
    of the group through CUDA IPC.  ``ptrs[r]`` is the address of rank r's buffer in this process."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        lib = ops.lib()
        self.nbytes, self.rank, self.world = int(nbytes), rank, world
        self._local = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        ops.check(lib.rlz_symm_alloc(self.nbytes, ctypes.byref(self._local), handle), "symm_alloc")
        handles: List[Optional[bytes]] = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        else:
            handles[0] = handle.raw
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self._local.value)
                continue
            p = ctypes.c_void_p()
            ops.check(lib.rlz_symm_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(p)), f"symm_open(rank {r})")
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        if world > 1:
            dist.barrier(group=group)

    def close(self):
        lib = ops.lib()
        for p in self._opened:
            lib.rlz_symm_close(ctypes.c_void_p(p))
        self._opened = []
        if self._local and self._local.value:
            lib.rlz_symm_free(self._local)
            self._local = ctypes.c_void_p()


class TpCommBase:
    mode = "base"

    def __init__(self, rank: int, world: int, device):
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.fused = False

    # hooks used by the decode plan ---------------------------------------------------------
    def begin_step(self) -> None:
        """Issued once at the start of every step (before the first collective)."""

    def step_launches(self) -> int:
        return 0

    def ar_desc(self, site: int):
        return None

    def close(self):
        pass


class NcclTpComm(TpCommBase):
    mode = "nccl"

    def __init__(self, rank, world, device, group=None):
        super().__init__(rank, world, device)
        self.group = group

    def all_reduce_sum_(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def select_greedy(self, local_val: torch.Tensor, local_idx: torch.Tensor, out_idx: torch.Tensor, batch: int) -> None:
        """local (value, global token id) per batch row -> global argmax in ``out_idx``."""
        pair = torch.stack([local_val[:batch], local_idx[:batch].to(torch.float32)], dim=1).contiguous()
        allp = torch.empty(self.world, batch, 2, device=self.device, dtype=torch.float32)
        dist.all_gather_into_tensor(allp, pair, group=self.group)
        best = allp[:, :, 0].argmax(dim=0)
        out_idx[:batch] = allp[best, torch.arange(batch, device=self.device), 1].to(torch.int32)

    def gather_logits(self, local_logits: torch.Tensor, vocab: int) -> torch.Tensor:
        """[batch, vocab_local] on every rank -> [batch, vocab] (rank-major concatenation)."""
        b, vl = local_logits.shape
        allp = torch.empty(self.world, b, vl, device=self.device, dtype=local_logits.dtype)
        dist.all_gather_into_tensor(allp, local_logits.contiguous(), group=self.group)
        return allp.permute(1, 0, 2).reshape(b, self.world * vl)[:, :vocab].contiguous()


class FusedTpComm(NcclTpComm):
    """In-kernel collectives over symmetric peer memory (NCCL is kept only for set-up and for the
    non-greedy logits gather)."""
    mode = "fused"

    def __init__(self, rank, world, device, group=None, spin_limit: int = 20_000_000):
        super().__init__(rank, world, device, group)
        self.fused = True
        self.spin_limit = spin_limit
        self.buf: Optional[SymmetricBuffer] = None
        self.epoch = torch.zeros(1, device=self.device, dtype=torch.int32)
        self.status = torch.zeros(1, device=self.device, dtype=torch.int32)
        self._sites = []
        self._cand = None

    def allocate(self, n_sites: int, n: int, max_batch: int, max_ctas: int = 0) -> None:
        """Reserve symmetric memory for ``n_sites`` all-reduce call sites of ``n`` outputs each and
        for the candidate exchange of up to ``max_batch`` sequences."""
        w = self.world
        n_pad = (n + 3) // 4 * 4
        self.n, self.max_batch = n_pad, max_batch
        self._inbox_site = 2 * w * 4 * n_pad * 8           # [parity][rank][4 batch rows][n] pairs of 32-bit words
        self._off_cand = n_sites * self._inbox_site
        cand_inbox = 2 * w * max_batch * 2 * 8
        total = (self._off_cand + cand_inbox + 255) // 256 * 256
        if self.buf is not None:                           # a second engine on the same communicator: the first one's buffers go
            self.buf.close()
        self._cand = None
        self.buf = SymmetricBuffer(total, self.rank, w, self.group)
        self.n_sites = n_sites

    def ar_desc(self, site: int) -> S.GemvAr:
        if not 0 <= site < self.n_sites:
            raise IndexError(f"all-reduce site {site} out of range ({self.n_sites} reserved)")
        ar = S.GemvAr()
        for r in range(self.world):
            ar.inbox[r] = self.buf.ptrs[r] + site * self._inbox_site
        ar.epoch, ar.status = self.epoch.data_ptr(), self.status.data_ptr()
        ar.spin_limit = self.spin_limit
        ar.rank, ar.world, ar.enabled, ar.n = self.rank, self.world, 1, self.n
        return ar

    # -- row-parallel GEMMs of token batches (batched decode, short prompt chunks) -------------------
    def allocate_gemm(self, n_sites: int, n: int, max_tokens: int, splits: int = 4) -> None:
        """Symmetric inbox for row-parallel GEMMs of up to ``max_tokens`` x ``n`` outputs at ``n_sites`` call sites
        per pass: two alternating buffers of ``[world * splits writers][max_tokens][n]`` 8-byte {value, tag} pairs."""
        if n_sites > 256:
            raise ValueError("at most 256 GEMM all-reduce sites per pass")
        self.g_n = (n + 3) // 4 * 4
        self.g_rows, self.g_sites, self.g_splits = max_tokens, n_sites, splits
        self.gbuf = SymmetricBuffer(2 * self.world * splits * self.g_rows * self.g_n * 8, self.rank, self.world, self.group)

    def gemm_ar_fill(self, p: "S.GemmParams", site: int) -> None:
        """Turn a GEMM launch into "push my partial tiles to every rank" for call site ``site`` of the pass."""
        if not 0 <= site < self.g_sites:
            raise IndexError(f"GEMM all-reduce site {site} out of range ({self.g_sites} reserved)")
        for r in range(self.world):
            p.ar_inbox[r] = self.gbuf.ptrs[r]
        p.ar_epoch = self.epoch.data_ptr()
        p.ar_row_pairs, p.ar_rank, p.ar_world, p.ar_rows, p.ar_enabled = self.g_n, self.rank, self.world, self.g_rows, 1
        p.ar_site, p.ar_nsites, p.ar_splits = site, self.g_sites, self.g_splits
        p.splitk = min(self.g_splits, max(1, p.k // 64))

    def ll_reduce(self, site: int, x: torch.Tensor, tokens: int, n: int, k: int) -> None:
        """``x[:tokens, :n] += sum over ranks and K splits`` of what the GEMMs of call site ``site`` pushed (bounded polls)."""
        ops.check(ops.lib().rlz_ll_reduce(self.gbuf.ptrs[self.rank], self.epoch.data_ptr(), self.status.data_ptr(), self.spin_limit,
                                          self.world * self.g_splits, self.g_rows, self.g_n, site, self.g_sites, tokens, n, x.data_ptr(),
                                          x.stride(0), ops.stream_ptr()), "ll_reduce")

    # -- two-shot all-reduce of row-parallel GEMMs: reduce-scatter by row ownership, owner-side reduce + norm, all-gather ----
    def allocate_two_shot(self, n_sites: int, n: int, max_tokens: int, splits: int = 2) -> None:
        """Symmetric memory for the two-shot all-reduce of row-parallel GEMMs with up to ``max_tokens`` x ``n`` outputs at
        ``n_sites`` call sites per pass: the reduce-scatter inbox and tile flags, the all-gather flags, and the two buffers
        that finished rows are sent to - the bf16 operand ``xb`` and the fp32 residual stream ``x`` (views in ``ts_xb`` /
        ``ts_x``).  Token row t is owned by rank ``t // own_rows`` with ``own_rows = ceil(tokens / world)`` per call."""
        if n_sites > 256:
            raise ValueError("at most 256 all-reduce sites per pass")
        w = self.world
        a256 = lambda v: (v + 255) // 256 * 256
        self.ts_n = (n + 3) // 4 * 4
        self.ts_tokens, self.ts_sites, self.ts_splits = max_tokens, n_sites, splits
        self.ts_own_cap = -(-max_tokens // w)
        self.ts_ntiles, self.ts_mtiles = -(-n // 128), -(-max_tokens // 32)
        self._ts_off_inbox = 0
        off = a256(2 * w * splits * self.ts_own_cap * self.ts_n * 4)
        self._ts_off_flags = off
        off += a256(2 * w * splits * self.ts_ntiles * self.ts_mtiles * 4)
        self._ts_off_ag = off
        off += a256(w * self.ts_own_cap * 4)
        self._ts_off_x = off
        off += a256(max_tokens * self.ts_n * 4)
        self._ts_off_xb = off
        off += a256(max_tokens * self.ts_n * 2)
        self.tsbuf = SymmetricBuffer(off, self.rank, w, self.group)
        base = self.tsbuf.ptrs[self.rank]
        self.ts_x = _device_view(base + self._ts_off_x, max_tokens * self.ts_n * 4, self.device).view(torch.float32).view(max_tokens, self.ts_n)
        self.ts_xb = _device_view(base + self._ts_off_xb, max_tokens * self.ts_n * 2, self.device).view(torch.bfloat16).view(max_tokens, self.ts_n)

    def two_shot_fill(self, p: "S.GemmParams", site: int, tokens: int) -> None:
        """Turn a GEMM launch into the first half of the two-shot all-reduce at call site ``site`` of the pass: every tile
        goes to the inbox of the rank that owns its token rows, tagged per tile."""
        if not 0 <= site < self.ts_sites:
            raise IndexError(f"all-reduce site {site} out of range ({self.ts_sites} reserved)")
        if tokens > self.ts_tokens or p.n > self.ts_n:
            raise ValueError("GEMM exceeds the reserved two-shot buffers")
        for r in range(self.world):
            p.ar_inbox[r] = self.tsbuf.ptrs[r] + self._ts_off_inbox
            p.rs_flags[r] = self.tsbuf.ptrs[r] + self._ts_off_flags
        p.ar_epoch = self.epoch.data_ptr()
        p.ar_row_pairs, p.ar_rank, p.ar_world, p.ar_rows, p.ar_enabled = self.ts_n, self.rank, self.world, self.ts_own_cap, 2
        p.ar_site, p.ar_nsites, p.ar_splits = site, self.ts_sites, self.ts_splits
        p.rs_own_rows, p.rs_ntiles, p.rs_mtiles = -(-tokens // self.world), self.ts_ntiles, self.ts_mtiles
        p.splitk = max(1, min(p.splitk, self.ts_splits))

    def two_shot_reduce(self, p: "S.GemmParams", site: int, tokens: int, norm: int, nw, nb, eps: float, to_xb: bool, push_x: bool,
                        wait: bool = True) -> None:
        """Second half, for the GEMM described by ``p`` (after ``two_shot_fill``): the owner of each token row sums the
        partial rows onto its fp32 residual row, applies the norm that follows and sends the bf16 row to every rank's
        ``ts_xb`` (``to_xb``) and / or the fp32 row to every rank's ``ts_x`` (``push_x``); returns, on the stream, once the
        rows of all owners have arrived on this rank (``wait``)."""
        from ..ops import gemm as G
        nt, rows, sk = G.gemm_plan(p)
        c = S.RsReduce()
        base = self.tsbuf.ptrs[self.rank]
        c.inbox, c.flags = base + self._ts_off_inbox, base + self._ts_off_flags
        for r in range(self.world):
            c.ag_flags[r] = self.tsbuf.ptrs[r] + self._ts_off_ag
            c.xb[r] = self.tsbuf.ptrs[r] + self._ts_off_xb if to_xb else None
            c.xpeer[r] = self.tsbuf.ptrs[r] + self._ts_off_x
        c.x, c.nw, c.nb = base + self._ts_off_x, ops.ptr(nw), ops.ptr(nb)
        c.epoch, c.status, c.spin_limit = self.epoch.data_ptr(), self.status.data_ptr(), self.spin_limit
        c.ldx = c.ldxb = c.ld_in = self.ts_n
        c.rank, c.world, c.splits_stride, c.splits_used = self.rank, self.world, self.ts_splits, sk
        c.rows_cap = c.own_cap = self.ts_own_cap
        c.own_rows, c.tokens, c.n, c.nt = -(-tokens // self.world), tokens, p.n, nt
        c.n_tiles, c.ntiles_cap, c.mtiles_cap = -(-p.n // rows), self.ts_ntiles, self.ts_mtiles
        c.site, c.nsites, c.norm, c.push_x, c.wait_ag, c.eps = site, self.ts_sites, norm, 1 if push_x else 0, 1 if wait else 0, eps
        ops.check(ops.lib().rlz_rs_reduce(ctypes.byref(c), ops.stream_ptr()), "rs_reduce")

    # -- sampling with a vocabulary-sharded head: per-rank candidates, exchange over peer memory, same draw everywhere -------
    def allocate_sample(self, max_batch: int, k: int = 1024) -> None:
        """Symmetric memory for the candidate exchange of non-greedy sampling: per (parity, writer rank, sequence) ``k``
        {value, token id} pairs and one flag word."""
        w = self.world
        self.sm_k, self.sm_batch = k, max_batch
        pairs = 2 * w * max_batch * k * 8
        self._sm_off_flags = (pairs + 255) // 256 * 256
        if getattr(self, "sbuf", None) is not None:
            self.sbuf.close()
        self.sbuf = SymmetricBuffer(self._sm_off_flags + (2 * w * max_batch * 4 + 255) // 256 * 256, self.rank, w, self.group)

    def shard_sample_desc(self, index_offset: int) -> "S.ShardSample":
        c = S.ShardSample()
        for r in range(self.world):
            c.inbox[r] = self.sbuf.ptrs[r]
            c.flags[r] = self.sbuf.ptrs[r] + self._sm_off_flags
        c.epoch, c.status, c.spin_limit = self.epoch.data_ptr(), self.status.data_ptr(), self.spin_limit
        c.rank, c.world, c.batch_cap, c.K, c.index_offset = self.rank, self.world, self.sm_batch, self.sm_k, index_offset
        return c

    def sample_sharded(self, sp_local: "S.SampleParams", desc: "S.ShardSample") -> None:
        """``sp_local`` describes this rank's logits slice; the chosen token ids (identical on every rank) go to ``sp_local.out``."""
        lib = ops.lib()
        ops.check(lib.rlz_sample_push(ctypes.byref(sp_local), ctypes.byref(desc), ops.stream_ptr()), "sample_push")
        ops.check(lib.rlz_sample_merge(ctypes.byref(sp_local), ctypes.byref(desc), ops.stream_ptr()), "sample_merge")

    def begin_step(self) -> None:
        ops.check(ops.lib().rlz_epoch_bump(self.epoch.data_ptr(), ops.stream_ptr()), "epoch_bump")

    def step_launches(self) -> int:
        return 1

    def select_greedy(self, local_val, local_idx, out_idx, batch: int) -> None:
        if self._cand is None:
            c = S.CandExchange()
            for r in range(self.world):
                c.inbox[r] = self.buf.ptrs[r] + self._off_cand
            c.epoch, c.status, c.spin_limit = self.epoch.data_ptr(), self.status.data_ptr(), self.spin_limit
            c.rank, c.world, c.max_batch = self.rank, self.world, self.max_batch
            self._cand = c
        c = self._cand
        c.batch = batch
        ops.check(ops.lib().rlz_cand_exchange(ctypes.byref(c), local_val.data_ptr(), local_idx.data_ptr(), out_idx.data_ptr(), None,
                                              ops.stream_ptr()), "cand_exchange")

    def check_status(self) -> int:
        """Error code recorded by a kernel whose peer wait expired (0 = healthy)."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v

    def close(self):
        if self.buf is not None:
            self.buf.close()
            self.buf = None
        if getattr(self, "gbuf", None) is not None:
            self.gbuf.close()
            self.gbuf = None
        if getattr(self, "sbuf", None) is not None:
            self.sbuf.close()
            self.sbuf = None
        if getattr(self, "tsbuf", None) is not None:
            self.ts_x = self.ts_xb = None
            self.tsbuf.close()
            self.tsbuf = None


def make_tp_comm(rank: int, world: int, device, mode: str = "fused", group=None) -> TpCommBase:
    if mode == "nccl":
        return NcclTpComm(rank, world, device, group)
    if mode == "fused":
        return FusedTpComm(rank, world, device, group)
    raise ValueError(f"unknown tensor-parallel communication mode '{mode}'")
