"""Ring-buffer KV cache for unbounded streams: keeps the most recent ``window`` positions (plus
optional attention-sink positions at the start), fp32 or fp16 storage, O(1) append.
Host / torch reference structure (the serving engine uses the paged cache with a sliding window
in the attention kernel).  Reference parity: ``StreamingKVCache`` / ``StreamingKVCacheFp16``
(src/gpu/streaming_kv.rs:28-190)."""
from __future__ import annotations

from typing import Tuple

import torch


class StreamingKVCache:
    def __init__(self, num_layers: int, window: int, kv_heads: int, head_dim: int, sinks: int = 0, dtype=torch.float32, device="cpu"):
        if window <= sinks:
            raise ValueError("window must exceed the number of sink positions")
        self.L, self.window, self.sinks = num_layers, window, sinks
        self.k = torch.zeros(num_layers, window, kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.length = [0] * num_layers          # tokens ever appended per layer

    def _slot(self, t: int) -> int:
        if t < self.window:
            return t
        ring = self.window - self.sinks
        return self.sinks + (t - self.sinks) % ring

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> int:
        t = self.length[layer]
        s = self._slot(t)
        self.k[layer, s] = k.to(self.k.dtype)
        self.v[layer, s] = v.to(self.v.dtype)
        self.length[layer] = t + 1
        return s

    def valid(self, layer: int) -> int:
        return min(self.length[layer], self.window)

    def get(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(K, V, absolute positions) of the retained tokens in temporal order."""
        n, t = self.valid(layer), self.length[layer]
        if t <= self.window:
            pos = torch.arange(n)
            return self.k[layer, :n], self.v[layer, :n], pos
        ring = self.window - self.sinks
        recent = torch.arange(t - ring, t)
        slots = torch.cat([torch.arange(self.sinks), torch.tensor([self._slot(int(p)) for p in recent], dtype=torch.long)])
        pos = torch.cat([torch.arange(self.sinks), recent])
        return self.k[layer, slots], self.v[layer, slots], pos

    def memory_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def reset(self) -> None:
        self.length = [0] * self.L


def StreamingKVCacheFp16(num_layers: int, window: int, kv_heads: int, head_dim: int, sinks: int = 0, device="cpu") -> StreamingKVCache:
    return StreamingKVCache(num_layers, window, kv_heads, head_dim, sinks, torch.float16, device)
