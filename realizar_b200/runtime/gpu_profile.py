"""Per-device launch policy: which kernel path each operation takes and with what grid, derived
from the device properties and overridable through environment variables (one place instead of
scattered constants).  Reference parity: ``GpuProfile`` (src/cuda/gpu_profile.rs:1-280: kernel
variant selection by compute capability, warps per block, thresholds, env overrides)."""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass
from typing import Optional


@dataclass
class GpuProfile:
    name: str = "cpu"
    compute_capability: tuple = (0, 0)
    sm_count: int = 0
    memory_bytes: int = 0
    l2_bytes: int = 0
    # decode
    gemv_threads: int = 512
    gemv_ctas_per_sm_batch1: int = 2        # register path holds 2 CTAs of 512 threads per SM
    gemv_max_rows_per_launch: int = 4
    gemv_stream_variant: bool = False       # TMA-streamed GEMV (measured slower; opt-in)
    overlap_mlp_up: bool = False            # side-stream overlap of the MLP up-projection (measured slower; opt-in)
    pdl: bool = True                        # programmatic dependent launch
    cuda_graphs: bool = True
    attn_max_cluster_splits: int = 8        # split merge through cluster shared memory up to this many splits
    # token batches
    gemm_decode_min_batch: int = 16         # decode batches at least this large use the tensor-core GEMM
    batched_prefill_min: int = 8
    prefill_chunk: int = 512
    flash_prefill_min_tokens: int = 16
    tensor_cores: str = "none"              # "tcgen05" on sm_100

    @classmethod
    def detect(cls, device: Optional[int] = None, env: Optional[dict] = None) -> "GpuProfile":
        import torch
        e = os.environ if env is None else env
        p = cls()
        if torch.cuda.is_available():
            d = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
            p.name, p.compute_capability, p.sm_count, p.memory_bytes = d.name, (d.major, d.minor), d.multi_processor_count, d.total_memory
            p.l2_bytes = getattr(d, "L2_cache_size", 0)
            p.tensor_cores = "tcgen05" if d.major == 10 else "unsupported"
        p.gemv_stream_variant = e.get("RLZ_GEMV_STREAM", "0") == "1"
        p.overlap_mlp_up = e.get("RLZ_OVERLAP_UP", "0") == "1"
        p.pdl = e.get("RLZ_PDL", "1") != "0"
        p.cuda_graphs = e.get("RLZ_CUDA_GRAPHS", "1") != "0"
        for key, attr in (("RLZ_GEMM_DECODE_MIN_BATCH", "gemm_decode_min_batch"), ("RLZ_PREFILL_CHUNK", "prefill_chunk"),
                          ("RLZ_BATCHED_PREFILL_MIN", "batched_prefill_min")):
            if key in e:
                setattr(p, attr, int(e[key]))
        return p

    @property
    def supported(self) -> bool:
        """The CUDA kernels are built for sm_100a only."""
        return self.compute_capability[0] == 10

    def gemv_target_ctas(self, batch: int) -> int:
        return self.sm_count * (self.gemv_ctas_per_sm_batch1 if batch <= 1 else 1)

    def attn_splits(self, kv_heads: int, batch: int) -> int:
        want = max(1, (2 * max(1, self.sm_count)) // max(1, kv_heads * max(1, batch)))
        s = 1
        while s * 2 <= min(self.attn_max_cluster_splits, want):
            s *= 2
        return s

    def engine_config_overrides(self) -> dict:
        return {"pdl": self.pdl, "cuda_graphs": self.cuda_graphs, "gemm_decode_min_batch": self.gemm_decode_min_batch,
                "prefill_chunk": self.prefill_chunk, "batched_prefill_min": self.batched_prefill_min}

    def describe(self) -> dict:
        return asdict(self)
