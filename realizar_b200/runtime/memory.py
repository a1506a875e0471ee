"""Memory helpers around the engine: size-class pools of transient device buffers, pinned host
buffers and a staging pool for H2D/D2H traffic, the VRAM sufficiency check with the layer-streaming
plan for models that do not fit, a double-buffered layer streamer, and a CPU-vs-GPU dispatch
heuristic.  Reference parity: ``GpuMemoryPool`` / ``PinnedHostBuffer`` / ``StagingBufferPool`` /
``TransferMode`` (src/cuda/memory.rs:16-344), ``StreamingConfig`` / ``StreamingMode`` /
``check_vram_sufficient`` (src/cuda/streaming.rs:36-219), ``AsyncPipeline`` (src/cuda/pipeline.rs:24-292),
``HybridScheduler`` (src/gpu/scheduler), ``GpuBufferPool`` / ``CacheAlignedBuffer`` (src/gpu/mod.rs:41-125)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import torch


def size_class(nbytes: int, min_class: int = 256) -> int:
    """Round up to the next power of two (at least ``min_class``)."""
    c = min_class
    while c < nbytes:
        c <<= 1
    return c


@dataclass
class PoolStats:
    hits: int = 0
    misses: int = 0
    bytes_pooled: int = 0
    bytes_in_use: int = 0

    @property
    def hit_rate(self) -> float:
        t = self.hits + self.misses
        return self.hits / t if t else 0.0


class GpuMemoryPool:
    """Free lists of byte buffers per power-of-two size class on one device; ``acquire`` reuses a
    buffer of the class or allocates, ``release`` returns it; ``trim`` drops what is pooled."""

    def __init__(self, device="cpu", max_pooled_bytes: int = 1 << 30):
        self.device, self.max_pooled = torch.device(device), max_pooled_bytes
        self.free: Dict[int, List[torch.Tensor]] = {}
        self.stats = PoolStats()

    def acquire(self, nbytes: int) -> torch.Tensor:
        c = size_class(nbytes)
        lst = self.free.get(c)
        if lst:
            self.stats.hits += 1
            self.stats.bytes_pooled -= c
            t = lst.pop()
        else:
            self.stats.misses += 1
            t = torch.empty(c, dtype=torch.uint8, device=self.device)
        self.stats.bytes_in_use += c
        return t

    def release(self, t: torch.Tensor) -> None:
        c = t.numel()
        self.stats.bytes_in_use -= c
        if self.stats.bytes_pooled + c <= self.max_pooled:
            self.free.setdefault(c, []).append(t)
            self.stats.bytes_pooled += c

    def trim(self) -> int:
        n = self.stats.bytes_pooled
        self.free.clear()
        self.stats.bytes_pooled = 0
        return n


GpuBufferPool = GpuMemoryPool


class PinnedHostBuffer:
    """Page-locked host memory (falls back to pageable memory where pinning is unavailable)."""

    def __init__(self, nbytes: int):
        self.tensor = torch.empty(nbytes, dtype=torch.uint8)
        self.pinned = False
        if torch.cuda.is_available():
            try:
                self.tensor = self.tensor.pin_memory()
                self.pinned = True
            except RuntimeError:
                pass

    def view(self, dtype: torch.dtype, count: int) -> torch.Tensor:
        return self.tensor[: count * torch.empty((), dtype=dtype).element_size()].view(dtype)


class TransferMode(Enum):
    PAGEABLE = "pageable"
    PINNED = "pinned"
    ZERO_COPY = "zero_copy"


class StagingBufferPool:
    def __init__(self, buffer_bytes: int = 1 << 20, count: int = 4):
        self.buffers = [PinnedHostBuffer(buffer_bytes) for _ in range(count)]
        self.free = list(range(count))
        self.buffer_bytes = buffer_bytes

    def acquire(self) -> Optional[tuple]:
        if not self.free:
            return None
        i = self.free.pop()
        return i, self.buffers[i]

    def release(self, index: int) -> None:
        if index not in self.free:
            self.free.append(index)

    @property
    def mode(self) -> TransferMode:
        return TransferMode.PINNED if self.buffers and self.buffers[0].pinned else TransferMode.PAGEABLE


def cache_aligned_empty(count: int, dtype=torch.float32, alignment: int = 64) -> torch.Tensor:
    """Host tensor whose first element sits on an ``alignment``-byte boundary."""
    es = torch.empty((), dtype=dtype).element_size()
    raw = torch.empty(count * es + alignment, dtype=torch.uint8)
    off = (-raw.data_ptr()) % alignment
    return raw[off: off + count * es].view(dtype)


# -- does the model fit? -----------------------------------------------------------------------------
class StreamingMode(Enum):
    RESIDENT = "resident"            # everything on the device
    LAYER_STREAMING = "layer_streaming"   # weights in pinned host memory, two layer buffers on the device


@dataclass
class StreamingConfig:
    mode: StreamingMode
    weight_bytes: int
    kv_bytes: int
    workspace_bytes: int
    free_bytes: int
    layer_bytes: int = 0
    resident_layers: int = 0

    @property
    def required_bytes(self) -> int:
        return self.weight_bytes + self.kv_bytes + self.workspace_bytes


def check_vram_sufficient(weight_bytes: int, kv_bytes: int, free_bytes: int, num_layers: int, workspace_bytes: int = 256 << 20,
                          headroom: float = 0.05) -> StreamingConfig:
    """Resident if weights + KV + workspace fit in the free memory (minus headroom); otherwise plan
    layer streaming: as many layers resident as fit, the rest double-buffered from the host."""
    usable = int(free_bytes * (1 - headroom))
    if weight_bytes + kv_bytes + workspace_bytes <= usable:
        return StreamingConfig(StreamingMode.RESIDENT, weight_bytes, kv_bytes, workspace_bytes, free_bytes, weight_bytes // max(1, num_layers), num_layers)
    layer = -(-weight_bytes // max(1, num_layers))
    left = usable - kv_bytes - workspace_bytes - 2 * layer
    if left < 0:
        raise MemoryError(f"not enough device memory even with layer streaming: need {kv_bytes + workspace_bytes + 2 * layer} bytes, have {usable}")
    return StreamingConfig(StreamingMode.LAYER_STREAMING, weight_bytes, kv_bytes, workspace_bytes, free_bytes, layer, min(num_layers, left // layer))


class LayerStreamer:
    """Double-buffered prefetch: while layer ``i`` computes from one buffer, layer ``i+1`` is copied
    into the other on a side stream.  ``copy(layer, buffer_index)`` and ``compute(layer, buffer_index)``
    are supplied by the caller; with CUDA the copies run on their own stream and events order them.
    Stand-alone form of the schedule for callers that own their layers (``examples/stream_layers.py``); the engine's launch
    plans are built ahead of time, so ``models.decoder.GpuModel`` applies the same schedule through ``acquire_layer`` /
    ``release_layer`` hooks inside the plan."""

    def __init__(self, num_layers: int, copy: Callable[[int, int], None], compute: Callable[[int, int], None], use_cuda: Optional[bool] = None):
        self.n, self.copy, self.compute = num_layers, copy, compute
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.trace: List[tuple] = []

    def run(self) -> None:
        if not self.cuda:
            self.copy(0, 0); self.trace.append(("copy", 0, 0))
            for i in range(self.n):
                if i + 1 < self.n:
                    self.copy(i + 1, (i + 1) & 1); self.trace.append(("copy", i + 1, (i + 1) & 1))
                self.compute(i, i & 1); self.trace.append(("compute", i, i & 1))
            return
        main, side = torch.cuda.current_stream(), torch.cuda.Stream()
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        freed = [torch.cuda.Event(), torch.cuda.Event()]
        with torch.cuda.stream(side):
            self.copy(0, 0)
            ready[0].record(side)
        for i in range(self.n):
            b = i & 1
            if i + 1 < self.n:
                with torch.cuda.stream(side):
                    if i >= 1:
                        side.wait_event(freed[(i + 1) & 1])        # the buffer's previous layer has been consumed
                    self.copy(i + 1, (i + 1) & 1)
                    ready[(i + 1) & 1].record(side)
            main.wait_event(ready[b])
            self.compute(i, b)
            freed[b].record(main)


class ComputeBackend(Enum):
    CPU = "cpu"
    GPU = "gpu"
    AUTO = "auto"


@dataclass
class HybridScheduler:
    """CPU or GPU for one operation: the GPU wins when its compute advantage outweighs moving the
    operands over PCIe (transfer modelled at ``pcie_cost_factor`` x the GPU compute time per byte)."""
    gpu_available: bool = True
    min_gpu_elements: int = 1 << 16
    pcie_cost_factor: float = 5.0
    gpu_speedup: float = 20.0

    def choose(self, elements: int, operands_on_device: bool = False, preference: ComputeBackend = ComputeBackend.AUTO) -> ComputeBackend:
        if preference != ComputeBackend.AUTO:
            return preference if (preference == ComputeBackend.CPU or self.gpu_available) else ComputeBackend.CPU
        if not self.gpu_available or elements < self.min_gpu_elements:
            return ComputeBackend.CPU
        gpu_cost = elements / self.gpu_speedup * (1.0 if operands_on_device else 1.0 + self.pcie_cost_factor)
        return ComputeBackend.GPU if gpu_cost < elements else ComputeBackend.CPU


class GuardBands:
    """Allocator of zero-initialised tensors with canary bands: ``BAND`` bytes of a fixed pattern before and after every
    tensor (the tail up to the next 256-byte boundary included).  ``check()`` names the tensors whose bands changed: a kernel
    wrote outside the buffer it was given.  The engine allocates its step buffers through this when ``canaries`` is set and
    checks the bands in ``check_health()``.  Host-side stand-in for the guard pages a memory checker would give."""
    BAND = 256
    PATTERN = 0xA5

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.entries: List[tuple] = []                     # (name, raw uint8 tensor, payload bytes)

    def zeros(self, *shape, dtype=torch.float32, name: str = "") -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        raw = torch.full((2 * self.BAND + padded,), self.PATTERN, dtype=torch.uint8, device=self.device)
        raw[self.BAND: self.BAND + nbytes] = 0
        self.entries.append((name or f"buffer{len(self.entries)}", raw, nbytes))
        return raw[self.BAND: self.BAND + nbytes].view(dtype).view(*shape)

    def check(self) -> List[str]:
        """Names of the tensors with an overwritten band (one reduction per tensor; synchronises)."""
        bad = []
        for name, raw, nbytes in self.entries:
            front, back = raw[: self.BAND], raw[self.BAND + nbytes:]
            if bool((front != self.PATTERN).any()) or bool((back != self.PATTERN).any()):
                bad.append(name)
        return bad

    def bytes_reserved(self) -> int:
        return sum(int(raw.numel()) for _, raw, _ in self.entries)
