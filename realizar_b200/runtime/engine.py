"""Decode engine: static step buffers, the paged KV cache on the device, CUDA-graph capture of
the decode step per batch-size bucket, and slot-level sequence management.

One engine instance drives one GPU (one tensor-parallel rank).  The host never touches
activations: a step consumes ``tokens`` / ``positions`` / ``page_table`` that live on the
device and produces ``sampled`` token ids there; the streaming loop moves 4-byte ids through
pinned memory.

Capability parity with the reference's graph-captured decode (indirect position / seq_len
buffers, per-batch-size graphs; src/cuda/executor/layers/graphed_capture.rs:16-364,
src/cuda/executor/layers/forward_graphed_decode.rs:18-211) and with its batched decode state
(src/gguf/cuda/generate_batched_streaming.rs:8-660).
"""
from __future__ import annotations

import dataclasses
import logging
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..models.batched import BatchedForward, gemm_capable
from ..models.decoder import DecodePlan, GpuModel, StepBuffers, build_decode_plan, emit_head, emit_select
from ..ops import gemm as G
from ..models.weights import ModelWeights
from ..utils.trace import nvtx_range
from .paged_kv import PagedKvCache

log = logging.getLogger("realizar_b200.engine")

PAGE = 16
HISTORY_WINDOW = 64          # recent tokens per sequence that the repetition / presence / frequency penalties look at


@dataclass
class EngineConfig:
    max_batch: int = 4
    max_seq_len: int = 2048
    num_pages: Optional[int] = None        # default: enough for max_batch full-length sequences
    cuda_graphs: bool = True
    pdl: bool = True                       # programmatic dependent launch between kernels
    attn_splits: int = 0                   # 0 = choose from the SM count
    greedy_only: bool = False              # compile plans with argmax instead of the sampling kernel
    persistent_step: Optional[bool] = None # batch-1 step as one persistent cooperative kernel (None: RLZ_PERSISTENT, default off)
    prefill_chunk: int = 512               # tokens per tensor-core prefill pass
    batched_prefill_min: int = 8           # shorter prompts go through the decode kernels token by token
    gemm_decode_min_batch: int = 16        # decode batches at least this large run on the tensor-core GEMM path
    prefix_cache: bool = False             # share full KV pages between prompts with a common prefix
    parity_gate: bool = False              # at load: GPU vs CPU logits on the BOS token must agree (cosine >= 0.99)
    kv_dtype: str = "bf16"                 # "q8": int8 KV rows with a per-(token, head) scale (half the cache memory)
    resident_layers: Optional[int] = None  # layers whose matrices stay on the device; None = all if they fit, else as many as fit (the rest is streamed)
    canaries: bool = False                 # guard bands around every step buffer, inspected by check_health() (also RLZ_CANARIES=1)
    batch_buckets: Sequence[int] = ()      # graph buckets; default powers of two up to max_batch
    seed: int = 0


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    max_tokens: int = 64
    stop_token_ids: Sequence[int] = ()
    seed: Optional[int] = None
    repetition_penalty: float = 1.0        # > 1 discourages tokens of the recent history (divide positive / multiply negative logits)
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Optional[Dict[int, float]] = None     # token id -> additive bias (OpenAI logit_bias)


@dataclass
class Slot:
    seq_id: int = -1
    active: bool = False
    position: int = -1          # position of the token fed in the next step
    n_pages: int = 0
    history: Optional[List[int]] = None    # prompt tokens seen so far (prefix cache only)


class DecodeEngine:
    def __init__(self, weights: ModelWeights, config: Optional[EngineConfig] = None, device="cuda", comm=None,
                 tp_rank: int = 0, tp_size: int = 1):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DecodeEngine runs on a CUDA device; use models.cpu_model.CpuModel on the CPU")
        # launch policy of this device (grids, thresholds, environment overrides) in one place; an engine built without an explicit
        # configuration takes its defaults from it
        from .gpu_profile import GpuProfile
        self.profile = GpuProfile.detect(self.device.index if self.device.index is not None else torch.cuda.current_device())
        if not self.profile.supported:
            raise RuntimeError(f"the CUDA kernels of this library are built for sm_100a; device '{self.profile.name}' is "
                               f"sm_{self.profile.compute_capability[0]}{self.profile.compute_capability[1]}")
        self.cfg = config or EngineConfig(**self.profile.engine_config_overrides())
        self.comm = comm
        resident = self.cfg.resident_layers
        if resident is None:
            # does the model fit next to its KV cache?  If not, keep as many layers resident as fit and stream the others from
            # pinned host memory through two device buffers (the plan of the reference's src/cuda/streaming.rs:36-219)
            from .memory import StreamingMode, check_vram_sufficient
            wc, c0 = weights.config, self.cfg
            pages = c0.num_pages or c0.max_batch * -(-c0.max_seq_len // PAGE)
            rowb = (wc.head_dim + 16) if c0.kv_dtype == "q8" else 2 * wc.head_dim
            kv_est = 2 * wc.num_layers * pages * (wc.num_kv_heads // max(1, tp_size)) * PAGE * rowb
            free_bytes, _t = torch.cuda.mem_get_info(self.device)
            try:
                plan = check_vram_sufficient(weights.total_bytes() // max(1, tp_size), kv_est, free_bytes, wc.num_layers)
            except MemoryError as e:
                raise RuntimeError(f"model does not fit on {self.profile.name} even with layer streaming: {e}") from None
            if plan.mode == StreamingMode.LAYER_STREAMING:
                resident = plan.resident_layers
                log.warning("weights + KV cache exceed the free device memory: %d of %d layers resident, the rest streamed from host memory",
                            resident, wc.num_layers)
        self.model = GpuModel(weights, self.device, tp_rank, tp_size, resident_layers=resident)
        if self.model.streaming:                             # copies on a side stream between launches: no captured graphs
            self.cfg = dataclasses.replace(self.cfg, cuda_graphs=False, persistent_step=False)
        self.mcfg = self.model.cfg
        m, c, dev = self.model, self.cfg, self.device
        self.sm_count = self.profile.sm_count
        B = c.max_batch
        self.max_pages_per_seq = -(-c.max_seq_len // PAGE)
        self.num_pages = c.num_pages or B * self.max_pages_per_seq
        hd = self.mcfg.head_dim
        # [2 (k,v), layers, pages, kv_heads, PAGE, head_dim] bf16
        from .memory import check_vram_sufficient
        row = (hd + 16) if c.kv_dtype == "q8" else 2 * hd
        kv_bytes = 2 * self.mcfg.num_layers * self.num_pages * m.kv_heads * PAGE * row
        free_bytes, _total = torch.cuda.mem_get_info(self.device)
        try:                                                 # the weights are on the device already: what is left must hold the cache
            check_vram_sufficient(0, kv_bytes, free_bytes, self.mcfg.num_layers)
        except MemoryError:
            raise RuntimeError(f"KV cache of {kv_bytes / 2**30:.1f} GiB ({self.num_pages} pages) does not fit the {free_bytes / 2**30:.1f} GiB "
                               f"left on {self.profile.name}: lower max_batch / max_seq_len / num_pages or use kv_dtype='q8'") from None
        self.kv = ops.kv_cache_alloc(self.mcfg.num_layers, self.num_pages, m.kv_heads, hd, dev, c.kv_dtype, PAGE)
        self.pages = PagedKvCache(self.num_pages, PAGE)
        self.splits = c.attn_splits or self._choose_splits(B)        # at the full batch; smaller buckets split the context further
        qkv_w = m.q_dim + 2 * m.kv_dim
        o_k = max(L.o.k for L in m.layers)
        d_k = max(L.down.k for L in m.layers)
        y1_w = (m.act_col0 + d_k + 256) if self.mcfg.parallel_residual else qkv_w
        # step buffers: plain zeros, or (canaries) tensors with guard bands on both sides that check_health() inspects
        self.guards = None
        if c.canaries or os.environ.get("RLZ_CANARIES", "0") != "0":
            from .memory import GuardBands
            self.guards = GuardBands(dev)
        _n = [0]

        def z(*s, dt=torch.float32):
            if self.guards is None:
                return torch.zeros(*s, device=dev, dtype=dt)
            _n[0] += 1
            return self.guards.zeros(*s, dtype=dt, name=f"step buffer {_n[0]} {tuple(s)} {str(dt).split('.')[-1]}")
        self.buckets = sorted(set(c.batch_buckets or [b for b in (1, 2, 4, 8, 16, 32, 64, 128) if b < B] + [B]))
        part, ctr = ops.attn_decode_scratch(max(b * self.splits_for(b) for b in self.buckets), m.heads, 1, hd, dev)
        # tokens and positions are the two rows of one buffer (and of one pinned host buffer), so a step uploads both with one copy
        tok_pos = torch.zeros(2, B, device=dev, dtype=torch.int32)
        tok_pos[1].fill_(-1)
        self.buf = StepBuffers(
            tokens=tok_pos[0], positions=tok_pos[1],
            page_table=z(B, self.max_pages_per_seq, dt=torch.int32), x=z(B, self.mcfg.hidden_dim), y1=z(B, y1_w),
            attn_out=z(B, o_k), act=z(B, d_k + 256), partial_out=z(B, self.mcfg.hidden_dim) if tp_size > 1 else None,
            logits=z(B, m.vocab_local if tp_size > 1 else self.mcfg.vocab_size), sampled=z(B, dt=torch.int32),
            temperature=z(B), top_k=z(B, dt=torch.int32), top_p=torch.ones(B, device=dev), min_p=z(B), uniform=z(B),
            attn_partial=part, attn_counters=ctr,
            local_val=z(B) if tp_size > 1 else None, local_idx=z(B, dt=torch.int32) if tp_size > 1 else None,
            logits_full=z(B, self.mcfg.vocab_size) if (tp_size > 1 and not c.greedy_only) else None,
            act_q=z(ops.act_block_bytes((d_k + 127) // 128 * 128), dt=torch.uint8))
        if not c.greedy_only:                              # sampling plans carry per-sequence logit controls
            b = self.buf
            b.history = torch.full((B, HISTORY_WINDOW), -1, device=dev, dtype=torch.int32)
            b.repetition, b.presence, b.frequency = torch.ones(B, device=dev), z(B), z(B)
            b.bias, b.bias_on = z(B, self.mcfg.vocab_size), z(B, dt=torch.int32)
        if comm is not None and getattr(comm, "fused", False):
            chunks_max = -(-B // 4)
            per_layer = 1 if self.mcfg.parallel_residual else 2
            comm.allocate(self.mcfg.num_layers * per_layer * chunks_max, self.mcfg.hidden_dim, max_batch=B)
            if not c.greedy_only:
                comm.allocate_sample(B)                    # candidate exchange of vocabulary-sharded sampling
        self.slots = [Slot() for _ in range(B)]
        self._slot_bias: Dict[int, dict] = {}
        self._bias_live: Dict[int, bool] = {}
        self._plans: Dict[int, DecodePlan] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._gen = torch.Generator(device=dev).manual_seed(c.seed)
        # pinned staging for the streaming loop (page-locked where the host allows it, pageable otherwise) and a pool for the
        # large transient device buffers of scoring passes
        from .memory import GpuMemoryPool, PinnedHostBuffer
        self.pool = GpuMemoryPool(dev, max_pooled_bytes=1 << 30)
        pinned = lambda *shape: PinnedHostBuffer(4 * int(np.prod(shape))).view(torch.int32, int(np.prod(shape))).zero_().view(*shape)
        self._h_tok_pos = pinned(2, B)
        self._h_tok_pos[1].fill_(-1)
        self._h_tokens, self._h_positions = self._h_tok_pos[0], self._h_tok_pos[1]
        self._d_tok_pos = tok_pos
        self._np_tokens, self._np_positions = self._h_tokens.numpy(), self._h_positions.numpy()     # cheap scalar writes
        self._h_sampled = pinned(B)
        self._h_table = pinned(B, self.max_pages_per_seq)
        self._next_seq = 0
        self.pdl = c.pdl
        ops.set_pdl(self.pdl)
        self.steps_run = 0
        self.health_check_every = 256
        self.gemm_ok = gemm_capable(self.model)
        self._batched: Optional[BatchedForward] = None
        self._head_plans: Dict[int, DecodePlan] = {}
        self.prefix_hits = self.prefix_tokens_reused = 0
        if c.parity_gate:
            cos = self.parity_check(weights)
            if not cos >= 0.99:
                raise RuntimeError(f"parity gate failed: GPU vs CPU logits cosine {cos:.4f} < 0.99")

    # -- configuration helpers --------------------------------------------------------------
    def _choose_splits(self, batch: int) -> int:
        return self.profile.attn_splits(self.model.kv_heads, batch)     # power of two up to the cluster size: splits merge through DSMEM

    def splits_for(self, bucket: int) -> int:
        """Context splits of the decode attention at this batch bucket: few sequences leave SMs idle unless each head's
        context is cut into more pieces (an engine sized for 64 sequences still decodes a single one with 8 splits)."""
        return self.cfg.attn_splits or int(os.environ.get("RLZ_ATTN_SPLITS", "0")) or self._choose_splits(bucket)

    def bucket_for(self, batch: int) -> int:
        for b in self.buckets:
            if b >= batch:
                return b
        raise ValueError(f"batch {batch} exceeds max_batch {self.cfg.max_batch}")

    # -- plans and graphs -------------------------------------------------------------------
    def plan(self, bucket: int) -> DecodePlan:
        if bucket not in self._plans and self._use_batched_step(bucket):
            self._plans[bucket] = self._batched_step_plan(bucket)
        if bucket not in self._plans:
            self._plans[bucket] = build_decode_plan(self.model, self.buf, self.kv[0], self.kv[1], bucket, self.splits_for(bucket), self.comm,
                                                    self.cfg.greedy_only, self.sm_count, persistent=self._persistent_ok(bucket))
        return self._plans[bucket]

    def _persistent_ok(self, bucket: int) -> bool:
        want = self.cfg.persistent_step
        if want is None:
            want = os.environ.get("RLZ_PERSISTENT", "0") != "0"
        return bool(want) and bucket == 1 and self.comm is None and self.cfg.kv_dtype != "q8"

    def kernels_per_step(self, bucket: int) -> int:
        p = self.plan(bucket)
        if self._use_batched_step(bucket):
            if self.batched().launches_per_pass == 0:
                p.run()
            return p.kernel_launches + self.batched().launches_per_pass + 5
        return p.kernel_launches

    def _capture(self, bucket: int) -> Optional[torch.cuda.CUDAGraph]:
        plan = self.plan(bucket)
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            plan.run()                      # warm-up outside capture (sets kernel attributes, loads modules)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(self.device)
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                plan.run()
            return g
        except Exception as e:  # pragma: no cover - depends on driver support
            if self.pdl:
                log.warning("graph capture with programmatic dependent launch failed (%s); retrying without it", e)
                self.pdl = False
                ops.set_pdl(False)
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    plan.run()
                return g
            raise

    def _batched_step_plan(self, bucket: int) -> DecodePlan:
        """Decode step for a large batch on the tensor-core path: every projection is one GEMM over
        all ``bucket`` rows (weights read once per step, not once per 4 rows), attention runs per row
        over its own page-table row, and the lm_head is a GEMM as well."""
        bf = self.batched()
        m, b, cfg = self.model, self.buf, self.mcfg
        norm_t = ops.NORM_LAYER if cfg.uses_layernorm else ops.NORM_RMS
        plan = DecodePlan(self.sm_count)
        B = bucket

        def body():
            bf.tokens[:B].copy_(b.tokens[:B])
            bf.positions[:B].copy_(b.positions[:B])
            ops.page_rows(b.page_table, b.positions, bf.page_rows, B, PAGE)
            x = bf.forward(B, b.page_table, shared_table=False)
            ops.norm_bf16(x, bf.xb[:B], m.out_norm_w, m.out_norm_b, norm_t, cfg.eps)
            G.gemm_launch(self._lm_head_gemm[B])
        self._lm_head_gemm = getattr(self, "_lm_head_gemm", {})
        self._lm_head_gemm[B] = G.build_gemm_params(m.lm_head, bf.xb, b.logits, B, bias=m.lm_head_b, ldy=b.logits.stride(0))
        plan.add(body, launches=0)
        emit_select(plan, m, b, 0, B, self.comm, self.cfg.greedy_only)
        return plan

    def _use_batched_step(self, bucket: int) -> bool:
        return self.gemm_ok and bucket >= self.cfg.gemm_decode_min_batch and bucket <= self.cfg.prefill_chunk

    def run_step(self, batch: int) -> None:
        """Issue one decode step for slots ``0..batch-1`` on the current stream."""
        bucket = self.bucket_for(batch)
        plan = self.plan(bucket)
        if plan.program is not None:
            # one cooperative launch (plus token selection when it is not an argmax): nothing for a graph to save
            plan.run()
            self.steps_run += 1
            if self.steps_run % 256 == 0:
                plan.program.check()
            return
        with nvtx_range("decode step"):                     # (a no-op unless RLZ_NVTX=1)
            if self.cfg.cuda_graphs:
                g = self._graphs.get(bucket)
                if g is None:
                    g = self._graphs[bucket] = self._capture(bucket)
                g.replay()
            else:
                self.plan(bucket).run()
        self.steps_run += 1
        if self.steps_run % self.health_check_every == 0:
            self.check_health()

    def check_health(self) -> None:
        """Read the status words that kernels set when a bounded wait runs out (a peer that never answered, a copy that never
        landed, a position past its page table) and raise, so that the caller stops using results computed from missing
        data.  Called every ``health_check_every`` steps and after every prompt pass; it synchronises the device."""
        code = ops.device_error(clear=True)
        if not code and self.comm is not None and hasattr(self.comm, "check_status"):
            code = self.comm.check_status()
        if code:
            raise ops.KernelError(f"a device-side check failed with status {code}: a bounded wait expired or an index left its range; "
                                  "results since the last check are not valid")
        if self.guards is not None:
            bad = self.guards.check()
            if bad:
                raise ops.KernelError("guard bands overwritten next to: " + "; ".join(bad))

    def profile_step(self, batch: int = 1, steps: int = 4) -> dict:
        """Per-operation timing of the decode step at this batch: the plan is run launch by launch (no graph) with every launch
        bracketed by CUDA events, ``steps`` times; returns ``{kind: {total_ms, count, avg_us, share}}`` sorted by share
        (the brick profile of the reference's executor, src/cuda/executor/ profiler hooks)."""
        from ..utils.trace import BrickProfiler
        plan = self.plan(self.bucket_for(batch))
        prof = BrickProfiler(cuda=True)
        plan.run()                                           # warm-up (kernel attributes, first touches)
        for _ in range(max(1, steps)):
            plan.run(profiler=prof)
        return prof.summary()

    def brick_report(self, batch: int = 1, steps: int = 4, efficiency: float = 0.5) -> dict:
        """The decode step as compute bricks with roofline budgets: the weight-streaming launches against ``weight bytes /
        (copy bandwidth x efficiency)``, attention against the cached K/V bytes of the open sequences, measured with
        ``profile_step``; names the bottleneck (largest time above its budget).  Role of the reference's brick budgets and
        bottleneck report (src/brick/mod.rs:47-442)."""
        from ..utils.bricks import ComputeBrick, TokenBudget, TransformerLayerBrick
        from ..utils.kernel_bench import peaks
        bw = peaks()["hbm_gbs"]
        prof = self.profile_step(batch, steps)
        ctx = sum(max(0, s.position) for s in self.slots[:batch] if s.active)
        kv_bytes = 2 * self.mcfg.num_layers * self.mcfg.num_kv_heads * self.mcfg.head_dim * ctx * (1 if self.cfg.kv_dtype == "q8" else 2)
        nbytes = {"gemv": self.model.weight_bytes(), "gemm": self.model.weight_bytes(), "attn": kv_bytes}
        bricks = []
        for kind, st in prof.items():
            b = ComputeBrick(kind, TokenBudget.from_bytes(max(1, nbytes.get(kind, 1)), bw, efficiency), bytes_moved=nbytes.get(kind, 0))
            b.record(1e3 * st["total_ms"] / max(1, steps))
            bricks.append(b)
        layer = TransformerLayerBrick(bricks)
        worst = layer.bottleneck()
        return {"bandwidth_gbs": bw, "efficiency": efficiency, "step_us": layer.total_actual_us(), "budget_us": layer.total_budget_us(),
                "bricks": {b.name: {"us_per_step": b.last_us, "budget_us": b.budget.us_per_token, "gbs": b.achieved_gbs(), "launches": prof[b.name]["count"] // max(1, steps)}
                           for b in bricks},
                "bottleneck": None if worst is None else {"brick": worst.brick, "gap": worst.gap, "share": worst.share}}

    def advance(self, batch: int) -> None:
        """Device-side feedback: sampled tokens become the next inputs, positions move on."""
        ops.advance_(self.buf.tokens[:batch], self.buf.sampled[:batch], self.buf.positions[:batch], limit=self.cfg.max_seq_len)

    # -- slots ---------------------------------------------------------------------------------
    def free_slots(self) -> List[int]:
        return [i for i, s in enumerate(self.slots) if not s.active]

    def open_slot(self, slot: int, reserve_tokens: int) -> int:
        """Bind a new sequence to ``slot`` and reserve KV pages for ``reserve_tokens`` tokens."""
        s = self.slots[slot]
        if s.active:
            raise RuntimeError(f"slot {slot} is busy")
        if reserve_tokens > self.cfg.max_seq_len:
            raise ValueError(f"sequence of {reserve_tokens} tokens exceeds max_seq_len {self.cfg.max_seq_len}")
        seq_id = self._next_seq
        self._next_seq += 1
        self.pages.add_sequence(seq_id)
        s.seq_id, s.active, s.position, s.n_pages = seq_id, True, 0, 0
        s.history = [] if self.cfg.prefix_cache else None
        self._ensure_pages(slot, reserve_tokens)
        return seq_id

    def _ensure_pages(self, slot: int, length: int) -> None:
        s = self.slots[slot]
        pages = self.pages.reserve(s.seq_id, length)
        if len(pages) != s.n_pages:
            row = self._h_table[slot]
            row[: len(pages)] = torch.tensor(pages, dtype=torch.int32)
            self.buf.page_table[slot].copy_(row, non_blocking=True)
            s.n_pages = len(pages)

    def close_slot(self, slot: int) -> None:
        s = self.slots[slot]
        if not s.active:
            return
        self.pages.free_sequence(s.seq_id)
        s.active, s.seq_id, s.position, s.n_pages = False, -1, -1, 0
        self._h_positions[slot] = -1
        self.buf.positions[slot: slot + 1].fill_(-1)
        if self.buf.history is not None:
            self.buf.history[slot].fill_(-1)
            if self._bias_live.get(slot):
                self.buf.bias_on[slot] = 0
                self._bias_live[slot] = False
            self._slot_bias.pop(slot, None)

    def set_sampling(self, slot: int, sp: SamplingParams) -> None:
        b = self.buf
        b.temperature[slot] = float(sp.temperature)
        b.top_k[slot] = int(sp.top_k)
        b.top_p[slot] = float(sp.top_p)
        b.min_p[slot] = float(sp.min_p)
        wants_controls = sp.repetition_penalty != 1.0 or sp.presence_penalty != 0.0 or sp.frequency_penalty != 0.0 or bool(sp.logit_bias)
        if b.history is None:
            if wants_controls:
                raise RuntimeError("penalties and logit_bias need an engine built with greedy_only=False")
            return
        b.repetition[slot] = float(sp.repetition_penalty)
        b.presence[slot] = float(sp.presence_penalty)
        b.frequency[slot] = float(sp.frequency_penalty)
        self._slot_bias[slot] = dict(sp.logit_bias or {})
        self._write_bias_row(slot, None)

    def _write_bias_row(self, slot: int, allowed) -> None:
        """Row ``slot`` of the additive logit row = the request's logit_bias entries, with -inf for every token outside
        ``allowed`` (a boolean vocabulary mask from a grammar, or None)."""
        b = self.buf
        lb = self._slot_bias.get(slot) or {}
        if allowed is None and not lb:
            if self._bias_live.get(slot):
                b.bias_on[slot] = 0
                self._bias_live[slot] = False
            return
        V = self.mcfg.vocab_size
        row = torch.zeros(V, dtype=torch.float32)
        if allowed is not None:
            m = torch.as_tensor(allowed[:V], dtype=torch.bool)
            if bool(m.any()):                              # an empty mask would leave nothing to sample: ignore it
                row[: m.numel()][~m] = float("-inf")
                row[m.numel():] = float("-inf")
        for t, v in lb.items():
            if 0 <= int(t) < V:
                row[int(t)] += float(v)
        b.bias[slot].copy_(row, non_blocking=False)
        b.bias_on[slot] = 1
        self._bias_live[slot] = True

    def set_token_mask(self, slot: int, allowed) -> None:
        """Restrict the next sampled token of ``slot`` to the ids where ``allowed`` (boolean array over the vocabulary) is
        true - the device-side form of a grammar / tool-call token mask; ``None`` lifts the restriction."""
        if self.buf.history is None:
            raise RuntimeError("token masks need an engine built with greedy_only=False")
        self._write_bias_row(slot, allowed)

    def _push_history(self, slot: int, tokens: Sequence[int], pos0: int) -> None:
        """Prompt tokens at positions ``pos0 ..`` enter the slot's history ring (decode steps add theirs on the device)."""
        if self.buf.history is None or not tokens:
            return
        W = HISTORY_WINDOW
        tail = list(tokens)[-W:]
        p0 = pos0 + len(tokens) - len(tail)
        idx = torch.tensor([(p0 + i) % W for i in range(len(tail))], dtype=torch.long, device=self.device)
        self.buf.history[slot, idx] = torch.tensor(tail, dtype=torch.int32, device=self.device)

    # -- single-token feeding ------------------------------------------------------------------
    def feed(self, slot_tokens: Dict[int, int]) -> torch.Tensor:
        """Run one step feeding ``{slot: token}`` at each slot's current position; other slots idle.
        Returns the pinned host tensor of sampled ids (valid after the implied synchronisation)."""
        hi = max(slot_tokens) + 1
        for i in range(hi):
            s = self.slots[i]
            if i in slot_tokens and s.active:
                self._ensure_pages(i, s.position + 1)
                self._np_tokens[i] = slot_tokens[i]
                self._np_positions[i] = s.position
            else:
                self._np_positions[i] = -1
        b = self.buf
        self._d_tok_pos.copy_(self._h_tok_pos, non_blocking=True)      # host state is authoritative in this loop: rows >= hi are idle (-1)
        if not self.cfg.greedy_only:
            b.uniform[:hi].copy_(torch.rand(hi, device=self.device, generator=self._gen))
        self.run_step(hi)
        self._h_sampled[:hi].copy_(b.sampled[:hi], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        for i in slot_tokens:
            if self.slots[i].active:
                self.slots[i].position += 1
        return self._h_sampled

    def batched(self) -> BatchedForward:
        if self._batched is None:
            self._batched = BatchedForward(self.model, self.cfg.prefill_chunk, self.kv[0], self.kv[1], self.max_pages_per_seq, self.comm, self.sm_count)
        return self._batched

    def _head(self, slot: int) -> DecodePlan:
        """Final norm + lm_head + token selection for one row of the step buffers."""
        if slot not in self._head_plans:
            plan = DecodePlan(self.sm_count)
            emit_head(plan, self.model, self.buf, slot, 1, self.comm, self.cfg.greedy_only, self.sm_count)
            self._head_plans[slot] = plan
        return self._head_plans[slot]

    def prefill(self, slot: int, tokens: Sequence[int]) -> int:
        """Run a prompt (or a prompt continuation) for ``slot`` and return the token sampled after its
        last token.  Prompts of at least ``batched_prefill_min`` tokens go through the tensor-core GEMM
        pass in chunks of ``prefill_chunk`` tokens when every projection supports it; otherwise the
        prompt is fed through the decode kernels token by token (as the reference's ``run_prefill``
        loop, src/gguf/cuda/generate_2.rs:261-273)."""
        s = self.slots[slot]
        if s.history is not None:
            tokens = list(tokens)
            if s.position == 0 and len(tokens) > PAGE:
                # swap the slot's fresh pages for cached ones that already hold this prompt's leading pages
                reserved = len(self.pages.seqs[s.seq_id].pages) * PAGE
                self.pages.rollback(s.seq_id, 0)
                covered = self.pages.match_prefix(s.seq_id, tokens)
                s.n_pages = -1
                self._ensure_pages(slot, max(reserved, len(tokens)))
                if covered:
                    self.prefix_hits += 1
                    self.prefix_tokens_reused += covered
                    s.position = covered
                    s.history = tokens[:covered]
                    tokens = tokens[covered:]
            s.history.extend(int(t) for t in tokens)
        n = len(tokens)
        if n >= self.cfg.batched_prefill_min and self.gemm_ok:
            self._push_history(slot, tokens, s.position)       # (the token-by-token path below records them on the device)
            out = self._prefill_batched(slot, tokens)
        else:
            out = 0
            for t in tokens:
                out = int(self.feed({slot: int(t)})[slot])
        if s.history is not None:
            self.pages.publish_prefix(s.seq_id, s.history)
        return out

    def parity_check(self, weights: ModelWeights, token: Optional[int] = None) -> float:
        """Cosine similarity of the logits of one token (BOS by default) between this engine and the
        C++ CPU engine on the same weights (the reference gates its CUDA model the same way,
        src/gguf/cuda/mod.rs parity gate)."""
        from ..models.cpu_model import CpuModel
        tok = token if token is not None else (self.mcfg.bos_token_id if self.mcfg.bos_token_id is not None else 1)
        cpu = CpuModel(weights, 16).forward(int(tok), 0)
        slot = self.free_slots()[0]
        self.open_slot(slot, 16)
        try:
            self.feed({slot: int(tok)})
            gpu = self.buf.logits[slot, : self.mcfg.vocab_size].float().cpu().numpy()
        finally:
            self.close_slot(slot)
        import numpy as np
        a, b = np.asarray(cpu, np.float64), np.asarray(gpu, np.float64)
        if self.model.tp_size > 1:                    # vocabulary-sharded lm_head: compare this rank's slice
            b = b[: self.model.vocab_local]
            a = a[self.model.vocab_start: self.model.vocab_start + b.shape[0]]
        return float(a @ b / max(1e-30, np.linalg.norm(a) * np.linalg.norm(b)))

    def _prefill_batched(self, slot: int, tokens: Sequence[int]) -> int:
        s = self.slots[slot]
        bf = self.batched()
        n, pos0 = len(tokens), s.position
        self._ensure_pages(slot, pos0 + n)
        pages = self.pages.seqs[s.seq_id].pages
        toks = torch.as_tensor(list(tokens), dtype=torch.int32)
        x_last = None
        for c0 in range(0, n, bf.T):
            T = min(bf.T, n - c0)
            pos = torch.arange(pos0 + c0, pos0 + c0 + T, dtype=torch.int32)
            rows = torch.tensor([pages[p // PAGE] for p in range(pos0 + c0, pos0 + c0 + T)], dtype=torch.int32)
            bf.tokens[:T].copy_(toks[c0:c0 + T], non_blocking=True)
            bf.positions[:T].copy_(pos, non_blocking=True)
            bf.page_rows[:T].copy_(rows, non_blocking=True)
            x = bf.forward_chunk(T, self.buf.page_table[slot], pos0 + c0)
            x_last = x[T - 1]
        self.buf.x[slot].copy_(x_last)
        if not self.cfg.greedy_only:
            self.buf.uniform[slot: slot + 1].copy_(torch.rand(1, device=self.device, generator=self._gen))
        self.buf.positions[slot: slot + 1].fill_(-1)         # the head plan's history update has nothing to add: the prompt is in already
        self._head(slot).run()
        self._h_sampled[slot: slot + 1].copy_(self.buf.sampled[slot: slot + 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.check_health()
        s.position = pos0 + n
        return int(self._h_sampled[slot])

    # -- multi-token verification / speculative support ------------------------------------------
    def forward_tokens(self, slot: int, tokens: Sequence[int]) -> List[int]:
        """Feed ``tokens`` at the slot's current position (KV appended) and return the greedy next
        token after EACH of them: one tensor-core pass over all rows plus one lm_head pass per
        ``max_batch`` rows.  Used to verify draft tokens in a single weight read
        (the reference verifies through its batched GEMV, src/gguf/cuda/speculative.rs:120-200)."""
        n = len(tokens)
        s = self.slots[slot]
        if n == 0:
            return []
        if not self.gemm_ok or n < 2:
            self.buf.temperature[slot] = 0.0
            return [int(self.feed({slot: int(t)})[slot]) for t in tokens]
        bf = self.batched()
        if n > bf.T:
            raise ValueError(f"{n} tokens exceed the batched-pass capacity {bf.T}")
        pos0 = s.position
        self._ensure_pages(slot, pos0 + n)
        pages = self.pages.seqs[s.seq_id].pages
        pos = torch.arange(pos0, pos0 + n, dtype=torch.int32)
        bf.tokens[:n].copy_(torch.as_tensor(list(tokens), dtype=torch.int32), non_blocking=True)
        bf.positions[:n].copy_(pos, non_blocking=True)
        bf.page_rows[:n].copy_(torch.tensor([pages[p // PAGE] for p in range(pos0, pos0 + n)], dtype=torch.int32), non_blocking=True)
        x = bf.forward_chunk(n, self.buf.page_table[slot], pos0)
        out: List[int] = []
        B = self.cfg.max_batch
        fused = self.comm is not None and getattr(self.comm, "fused", False)
        for c0 in range(0, n, B):
            cb = min(B, n - c0)
            if fused and c0 > 0:
                # the peer stores of the candidate exchange are tagged with the epoch alone: a second exchange needs a new
                # one, or a rank could read the previous chunk's pairs (same tag) before its peers have stored the new ones
                self.comm.begin_step()
            self.buf.x[:cb].copy_(x[c0:c0 + cb])
            key = ("verify", cb)
            if key not in self._head_plans:
                plan = DecodePlan(self.sm_count)
                emit_head(plan, self.model, self.buf, 0, cb, self.comm, True, self.sm_count)
                self._head_plans[key] = plan
            self._head_plans[key].run()
            out += [int(v) for v in self.buf.sampled[:cb].cpu()]
        s.position = pos0 + n
        return out

    # -- scoring: log-probabilities of given tokens, pooled embeddings ------------------------------------------
    def score_tokens(self, tokens: Sequence[int], want_embedding: bool = False, top_k: int = 0) -> dict:
        """Teacher-forced pass over ``tokens`` on the tensor-core path: ``logprobs[i] = log p(tokens[i+1] | tokens[:i+1])``
        for i = 0 .. n-2 (head GEMM over every row + a log-softmax / gather kernel), optionally the top-k alternatives at
        every position and the mean-pooled final-norm hidden state.  Uses a free slot for the duration of the call (run it on
        the engine thread).  Under tensor parallelism every rank calls it with the same tokens; the vocabulary-sharded head is
        combined with small all-reduces.  The reference computes these on the host from downloaded logits
        (``generate_gpu_resident_logprobs`` / ``perplexity_gpu_resident``, src/gguf/cuda/generate_2.rs:590-780)."""
        import math
        n = len(tokens)
        if n < 1:
            raise ValueError("score_tokens needs at least one token")
        if not self.gemm_ok:
            raise RuntimeError("scoring runs on the tensor-core token-batch path: every projection must be Q4_K / Q5_K / Q6_K / bf16 / f16")
        if n > self.cfg.max_seq_len:
            raise ValueError(f"{n} tokens exceed max_seq_len {self.cfg.max_seq_len}")
        free = self.free_slots()
        if not free:
            raise RuntimeError("no free slot for scoring")
        slot = free[-1]
        bf, m, cfg = self.batched(), self.model, self.mcfg
        norm_t = ops.NORM_LAYER if cfg.uses_layernorm else ops.NORM_RMS
        tp = m.tp_size > 1
        vloc = m.vocab_local if tp else cfg.vocab_size
        raw_logits = self.pool.acquire(bf.T * vloc * 4)      # chunk rows x vocabulary slice, fp32: back to the pool when the pass ends
        self._score_logits = raw_logits[: bf.T * vloc * 4].view(torch.float32).view(bf.T, vloc)
        toks = torch.as_tensor(list(tokens), dtype=torch.int32)
        lps: List[float] = []
        tops: List[list] = []
        pooled = torch.zeros(cfg.hidden_dim, device=self.device, dtype=torch.float32) if want_embedding else None
        self.open_slot(slot, n)
        try:
            s = self.slots[slot]
            pages = self.pages.seqs[s.seq_id].pages
            for c0 in range(0, n, bf.T):
                T = min(bf.T, n - c0)
                bf.tokens[:T].copy_(toks[c0:c0 + T], non_blocking=True)
                bf.positions[:T].copy_(torch.arange(c0, c0 + T, dtype=torch.int32), non_blocking=True)
                bf.page_rows[:T].copy_(torch.tensor([pages[p // PAGE] for p in range(c0, c0 + T)], dtype=torch.int32), non_blocking=True)
                x = bf.forward_chunk(T, self.buf.page_table[slot], c0)
                ops.norm_bf16(x, bf.xb[:T], m.out_norm_w, m.out_norm_b, norm_t, cfg.eps)
                if pooled is not None:
                    pooled += bf.xb[:T].float().sum(0)
                rows = min(T, n - 1 - c0)                   # the last token of the sequence has no successor to score
                if rows > 0:
                    G.gemm_launch(G.build_gemm_params(m.lm_head, bf.xb, self._score_logits, T, bias=m.lm_head_b, ldy=self._score_logits.stride(0)))
                    tgt = toks[c0 + 1: c0 + 1 + rows].to(self.device)
                    parts = ops.logprob_parts(self._score_logits[:rows], tgt, index_offset=m.vocab_start if tp else 0, vocab=vloc)
                    if tp:
                        import torch.distributed as dist
                        gmax = parts[:, 0].clone()
                        dist.all_reduce(gmax, op=dist.ReduceOp.MAX)
                        ssum = parts[:, 1] * torch.exp(parts[:, 0] - gmax)
                        dist.all_reduce(ssum)
                        tl = parts[:, 2].clone()
                        dist.all_reduce(tl, op=dist.ReduceOp.MAX)
                        lp = tl - gmax - torch.log(ssum)
                    else:
                        lp = parts[:, 2] - parts[:, 0] - torch.log(parts[:, 1])
                    lps += [float(v) for v in lp.cpu()]
                    if top_k > 0 and not tp:
                        lsm = torch.log_softmax(self._score_logits[:rows, :cfg.vocab_size], dim=-1)
                        tv, ti = lsm.topk(min(top_k, cfg.vocab_size), dim=-1)
                        tops += [[(int(i), float(v)) for i, v in zip(ri, rv)] for ri, rv in zip(ti.cpu(), tv.cpu())]
            self.check_health()
        finally:
            self.close_slot(slot)
            self._score_logits = None
            self.pool.release(raw_logits)
        out = {"logprobs": lps, "num_tokens": n}
        if lps:
            nll = -sum(lps) / len(lps)
            out.update({"nll": nll, "perplexity": math.exp(min(nll, 700.0))})
        if top_k > 0:
            out["top_logprobs"] = tops
        if pooled is not None:
            out["embedding"] = [float(v) for v in (pooled / n).cpu()]
        return out

    def rollback(self, slot: int, position: int) -> None:
        """Forget everything at and after ``position`` (rejected draft tokens): the pages past it
        go back to the pool and later appends overwrite the stale entries."""
        s = self.slots[slot]
        if not 0 <= position <= s.position:
            raise ValueError(f"rollback to {position} outside 0..{s.position}")
        self.pages.rollback(s.seq_id, position)
        s.position = position
        s.n_pages = -1                       # force a page-table refresh on the next reserve

    def draft_step(self, slot: int, token: int, layer_subset: Sequence[int]) -> int:
        """One greedy decode step of ``slot`` through a subset of the layers (shared KV cache)."""
        key = tuple(layer_subset)
        if not hasattr(self, "_draft_plans"):
            self._draft_plans: Dict[tuple, DecodePlan] = {}
        if key not in self._draft_plans:
            if slot != 0:
                raise ValueError("the layer-skipping draft runs in slot 0")
            self._draft_plans[key] = build_decode_plan(self.model, self.buf, self.kv[0], self.kv[1], 1, self.splits_for(1), self.comm, True,
                                                       self.sm_count, layer_subset=set(key))
        s = self.slots[slot]
        self._ensure_pages(slot, s.position + 1)
        self._h_tokens[slot] = int(token)
        self._h_positions[slot] = s.position
        self.buf.tokens[slot:slot + 1].copy_(self._h_tokens[slot:slot + 1], non_blocking=True)
        self.buf.positions[slot:slot + 1].copy_(self._h_positions[slot:slot + 1], non_blocking=True)
        self._draft_plans[key].run()
        s.position += 1
        return int(self.buf.sampled[slot].item())

    # -- convenience ----------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None, on_token=None) -> List[int]:
        """Generate for a single prompt in slot 0 (streams through ``on_token`` if given)."""
        sp = sampling or SamplingParams()
        free = self.free_slots()
        if not free:
            raise RuntimeError("no free slot")
        slot = free[0]
        self.open_slot(slot, min(self.cfg.max_seq_len, len(prompt) + sp.max_tokens))
        try:
            self.set_sampling(slot, sp)
            nxt = self.prefill(slot, prompt)
            out: List[int] = []
            stop = set(sp.stop_token_ids)
            for _ in range(sp.max_tokens):
                out.append(nxt)
                if on_token is not None:
                    on_token(nxt)
                if nxt in stop or self.slots[slot].position >= self.cfg.max_seq_len:
                    break
                nxt = int(self.feed({slot: nxt})[slot])
            return out
        finally:
            self.close_slot(slot)

    # -- KV snapshots (host-side prefix cache, migration between engines) ----------------------------
    def snapshot_kv(self, slot: int) -> dict:
        """Copy the slot's KV pages to pinned host memory.  Returns what ``restore_kv`` needs."""
        s = self.slots[slot]
        pages = list(self.pages.seqs[s.seq_id].pages[: self.pages.pages_needed(s.position)])
        idx = torch.tensor(pages, dtype=torch.long, device=self.device)
        data = self.kv[:, :, idx].to("cpu", non_blocking=False)
        return {"position": s.position, "pages": len(pages), "kv": data.pin_memory() if torch.cuda.is_available() else data}

    def restore_kv(self, slot: int, snap: dict) -> None:
        """Load a snapshot into a freshly opened slot (its pages may differ from the original ones)."""
        s = self.slots[slot]
        if s.position != 0:
            raise RuntimeError("restore_kv needs an empty slot")
        self._ensure_pages(slot, max(1, snap["position"]))
        pages = self.pages.seqs[s.seq_id].pages[: snap["pages"]]
        idx = torch.tensor(pages, dtype=torch.long, device=self.device)
        self.kv[:, :, idx] = snap["kv"].to(self.device, non_blocking=True)
        s.position = snap["position"]

    def reset(self) -> None:
        """Back to the post-load state after a failed step: probe the device (a lost context makes the synchronise raise, and
        then nothing in this process can use the GPU again), close every open sequence, clear the device-side status words and
        mark every row idle.  Weights, captured graphs and launch plans stay: they do not depend on sequence state."""
        torch.cuda.synchronize(self.device)                  # raises when the context is poisoned
        for slot, s in enumerate(self.slots):
            if s.active:
                self.close_slot(slot)
        ops.device_error(clear=True)
        if self.comm is not None and hasattr(self.comm, "check_status"):
            self.comm.check_status()
        self._h_tok_pos[1].fill_(-1)
        self.buf.positions.fill_(-1)
        self.steps_run = 0
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        """Release the captured graphs and launch plans (they hold kernels, buffers and, under tensor parallelism, work of the
        process group's communicator) and wait for the device.  Call before ``torch.distributed.destroy_process_group()``:
        a communicator that still has captured collectives alive can block its own destruction."""
        self._graphs.clear()
        self._plans.clear()
        self._head_plans.clear()
        if hasattr(self, "_draft_plans"):
            self._draft_plans.clear()
        self._batched = None
        torch.cuda.synchronize(self.device)

    def logits_of_last_step(self, slot: int = 0) -> torch.Tensor:
        return self.buf.logits[slot, : self.mcfg.vocab_size].clone()

    def memory_report(self) -> dict:
        return {"weights_bytes": self.model.weight_bytes(), "kv_bytes": self.kv.numel() * self.kv.element_size(), "kv_pages": self.num_pages,
                "kv_utilization": self.pages.stats().utilization, "device": self.profile.describe(),
                "pool": {"hits": self.pool.stats.hits, "misses": self.pool.stats.misses, "bytes_pooled": self.pool.stats.bytes_pooled},
                "streamed_layers": len(self.model.layers) - self.model.streamed_from}
