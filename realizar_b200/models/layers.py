"""Plain fp32 building blocks (PyTorch): LayerNorm, Linear, FeedForward, multi-head / multi-query /
grouped-query attention, fused-QKV attention, sliding-window attention, RoPE with context
scaling (linear, NTK, dynamic NTK, YaRN), ALiBi and a fused LayerNorm+Linear.  They are the
readable restatement that the oracle tests and small CPU models use; the serving path runs the
fused CUDA kernels instead.  Reference parity: src/layers/mod.rs (``LayerNorm``, ``Linear``,
``FeedForward``, ``Attention``, ``FusedQKVAttention``, ``SlidingWindowAttention``, ``RoPE``,
``ScaledRoPE``/``RopeScalingType``, ``ALiBi``, ``FusedLayerNormLinear``, ``Model``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


class LayerNorm(torch.nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight, self.bias, self.eps = torch.nn.Parameter(torch.ones(dim)), torch.nn.Parameter(torch.zeros(dim)), eps

    def forward(self, x):
        return F.layer_norm(x, x.shape[-1:], self.weight, self.bias, self.eps)


class RMSNorm(torch.nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight, self.eps = torch.nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.eps) * self.weight


class Linear(torch.nn.Module):
    def __init__(self, in_dim: int, out_dim: int, bias: bool = True, seed: Optional[int] = None):
        super().__init__()
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        self.weight = torch.nn.Parameter(torch.randn(out_dim, in_dim, generator=g) * in_dim ** -0.5)
        self.bias = torch.nn.Parameter(torch.zeros(out_dim)) if bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class FusedLayerNormLinear(torch.nn.Module):
    """``linear(layer_norm(x))`` with the normalisation folded into one pass over ``x``."""

    def __init__(self, in_dim: int, out_dim: int, eps: float = 1e-5):
        super().__init__()
        self.norm, self.linear = LayerNorm(in_dim, eps), Linear(in_dim, out_dim)

    def forward(self, x):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        w = self.linear.weight * self.norm.weight                       # fold gamma into the weight
        b = self.linear.bias + self.linear.weight @ self.norm.bias      # and beta into the bias
        return ((x - mu) * torch.rsqrt(var + self.norm.eps)) @ w.t() + b


class FeedForward(torch.nn.Module):
    def __init__(self, dim: int, hidden: int, gated: bool = False, activation: str = "gelu"):
        super().__init__()
        self.up, self.down = Linear(dim, hidden, bias=not gated), Linear(hidden, dim, bias=not gated)
        self.gate = Linear(dim, hidden, bias=False) if gated else None
        self.activation = activation

    def forward(self, x):
        act = F.gelu if self.activation == "gelu" else F.silu
        return self.down(act(self.gate(x)) * self.up(x)) if self.gate is not None else self.down(act(self.up(x)))


class RopeScalingType(Enum):
    NONE = "none"
    LINEAR = "linear"
    NTK = "ntk"
    DYNAMIC_NTK = "dynamic_ntk"
    YARN = "yarn"


@dataclass
class RopeScaling:
    kind: RopeScalingType = RopeScalingType.NONE
    factor: float = 1.0
    original_max_len: int = 2048
    beta_fast: float = 32.0
    beta_slow: float = 1.0


class RoPE:
    """Rotary embedding.  ``neox=False`` rotates adjacent pairs, ``neox=True`` split halves."""

    def __init__(self, dim: int, theta: float = 10000.0, neox: bool = False, scaling: Optional[RopeScaling] = None):
        self.dim, self.theta, self.neox, self.scaling = dim, theta, neox, scaling or RopeScaling()

    def inv_freq(self, seq_len: int = 0) -> Tuple[torch.Tensor, float]:
        """Per-pair frequencies and the attention ("mscale") factor for the configured scaling."""
        s, d = self.scaling, self.dim
        idx = torch.arange(0, d, 2, dtype=torch.float32) / d
        base = self.theta
        mscale = 1.0
        if s.kind == RopeScalingType.NTK:
            base = base * s.factor ** (d / (d - 2))
        elif s.kind == RopeScalingType.DYNAMIC_NTK and seq_len > s.original_max_len:
            a = s.factor * seq_len / s.original_max_len - (s.factor - 1)
            base = base * a ** (d / (d - 2))
        inv = base ** -idx
        if s.kind == RopeScalingType.LINEAR:
            inv = inv / s.factor
        elif s.kind == RopeScalingType.YARN:
            # blend interpolated (low-frequency) and original (high-frequency) bands
            def corr(n_rot):
                return d * math.log(s.original_max_len / (n_rot * 2 * math.pi)) / (2 * math.log(self.theta))
            lo, hi = max(math.floor(corr(s.beta_fast)), 0), min(math.ceil(corr(s.beta_slow)), d // 2 - 1)
            ramp = ((torch.arange(d // 2, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            inv = inv / s.factor * ramp + inv * (1 - ramp)
            mscale = 0.1 * math.log(s.factor) + 1.0 if s.factor > 1 else 1.0
        return inv, mscale

    def apply(self, x: torch.Tensor, positions: torch.Tensor, seq_len: int = 0) -> torch.Tensor:
        """``x`` [..., T, heads, head_dim]; rotates the first ``dim`` components of every head."""
        inv, mscale = self.inv_freq(seq_len or int(positions.max()) + 1)
        ang = positions.float()[:, None] * inv[None, :]
        cos, sin = (ang.cos() * mscale)[:, None, :], (ang.sin() * mscale)[:, None, :]
        rot, rest = x[..., : self.dim], x[..., self.dim:]
        if self.neox:
            a, b = rot[..., : self.dim // 2], rot[..., self.dim // 2:]
            out = torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
        else:
            a, b = rot[..., 0::2], rot[..., 1::2]
            out = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)
        return torch.cat([out, rest], -1)


ScaledRoPE = RoPE


class ALiBi:
    """Attention with linear biases: head ``h`` adds ``-slope_h * distance`` to its scores."""

    def __init__(self, num_heads: int):
        self.num_heads = num_heads
        n = 2 ** math.floor(math.log2(num_heads))
        base = [2 ** (-8.0 * (i + 1) / n) for i in range(n)]
        if n < num_heads:
            base += [2 ** (-4.0 * (2 * i + 1) / n) for i in range(num_heads - n)]
        self.slopes = torch.tensor(base)

    def bias(self, q_len: int, k_len: int) -> torch.Tensor:
        dist = (torch.arange(k_len)[None, :] - (torch.arange(q_len)[:, None] + (k_len - q_len))).clamp(max=0)
        return self.slopes[:, None, None] * dist[None].float()


class Attention(torch.nn.Module):
    """MHA (kv_heads = heads), GQA (1 < kv_heads < heads) or MQA (kv_heads = 1), causal, with an
    optional sliding window, RoPE or ALiBi, and an appendable KV cache."""

    def __init__(self, dim: int, heads: int, kv_heads: Optional[int] = None, head_dim: Optional[int] = None, rope: Optional[RoPE] = None,
                 alibi: bool = False, window: Optional[int] = None, bias: bool = False, fused_qkv: bool = False):
        super().__init__()
        self.heads, self.kv_heads = heads, kv_heads or heads
        self.hd = head_dim or dim // heads
        self.rope, self.window = rope, window
        self.alibi = ALiBi(heads) if alibi else None
        qd, kvd = heads * self.hd, self.kv_heads * self.hd
        self.fused = fused_qkv
        if fused_qkv:
            self.qkv = Linear(dim, qd + 2 * kvd, bias)
        else:
            self.q, self.k, self.v = Linear(dim, qd, bias), Linear(dim, kvd, bias), Linear(dim, kvd, bias)
        self.o = Linear(qd, dim, bias)

    def project(self, x):
        if self.fused:
            return self.qkv(x).split([self.heads * self.hd, self.kv_heads * self.hd, self.kv_heads * self.hd], -1)
        return self.q(x), self.k(x), self.v(x)

    def forward(self, x: torch.Tensor, cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """``x`` [T, dim] (new tokens).  Returns (out [T, dim], (K, V) cache with the new rows)."""
        T = x.shape[0]
        p0 = 0 if cache is None else cache[0].shape[0]
        q, k, v = self.project(x)
        q, k, v = q.view(T, self.heads, self.hd), k.view(T, self.kv_heads, self.hd), v.view(T, self.kv_heads, self.hd)
        pos = torch.arange(p0, p0 + T)
        if self.rope is not None:
            q, k = self.rope.apply(q, pos, p0 + T), self.rope.apply(k, pos, p0 + T)
        if cache is not None:
            k, v = torch.cat([cache[0], k]), torch.cat([cache[1], v])
        S = k.shape[0]
        rep = self.heads // self.kv_heads
        kh, vh = k.repeat_interleave(rep, 1).transpose(0, 1), v.repeat_interleave(rep, 1).transpose(0, 1)
        s = q.transpose(0, 1) @ kh.transpose(1, 2) * self.hd ** -0.5
        if self.alibi is not None:
            s = s + self.alibi.bias(T, S)
        kpos = torch.arange(S)
        mask = kpos[None, :] > pos[:, None]
        if self.window is not None:
            mask = mask | (kpos[None, :] <= pos[:, None] - self.window)
        s = s.masked_fill(mask[None], float("-inf"))
        out = (torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(T, -1)
        return self.o(out), (k, v)


    def forward_streaming(self, x: torch.Tensor, cache, layer: int = 0) -> torch.Tensor:
        """Token-by-token decoding over a ring-buffer cache (``runtime.streaming_kv.StreamingKVCache``): memory stays at
        ``cache.window`` positions however long the stream runs; every new token attends to the retained sink positions and the
        most recent ones, at their absolute positions.  With no sinks this equals ``forward`` with ``window = cache.window``.
        ``x`` [T, dim]; returns [T, dim]."""
        outs = []
        for t in range(x.shape[0]):
            q, k, v = self.project(x[t:t + 1])
            q, k, v = q.view(1, self.heads, self.hd), k.view(1, self.kv_heads, self.hd), v.view(1, self.kv_heads, self.hd)
            p = cache.length[layer]
            pos = torch.tensor([p])
            if self.rope is not None:
                q, k = self.rope.apply(q, pos, p + 1), self.rope.apply(k, pos, p + 1)
            cache.append(layer, k[0], v[0])
            ks, vs, kpos = cache.get(layer)
            rep = self.heads // self.kv_heads
            kh, vh = ks.float().repeat_interleave(rep, 1).transpose(0, 1), vs.float().repeat_interleave(rep, 1).transpose(0, 1)
            s = q.transpose(0, 1) @ kh.transpose(1, 2) * self.hd ** -0.5          # [heads, 1, retained]
            if self.alibi is not None:
                s = s - self.alibi.slopes[:, None, None] * (p - kpos)[None, None, :].float()
            outs.append((torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(1, -1))
        return self.o(torch.cat(outs))


def FusedQKVAttention(dim, heads, **kw):
    return Attention(dim, heads, fused_qkv=True, **kw)


def SlidingWindowAttention(dim, heads, window, **kw):
    return Attention(dim, heads, window=window, **kw)


class TransformerBlock(torch.nn.Module):
    def __init__(self, dim: int, heads: int, ffn: int, **attn_kw):
        super().__init__()
        self.n1, self.n2 = LayerNorm(dim), LayerNorm(dim)
        self.attn, self.ffn = Attention(dim, heads, **attn_kw), FeedForward(dim, ffn)

    def forward(self, x, cache=None):
        a, cache = self.attn(self.n1(x), cache)
        x = x + a
        return x + self.ffn(self.n2(x)), cache


class Model(torch.nn.Module):
    """Small decoder-only model assembled from the blocks above."""

    def __init__(self, vocab: int, dim: int, heads: int, layers: int, ffn: int, **attn_kw):
        super().__init__()
        self.embed = torch.nn.Embedding(vocab, dim)
        self.blocks = torch.nn.ModuleList([TransformerBlock(dim, heads, ffn, **attn_kw) for _ in range(layers)])
        self.norm, self.head = LayerNorm(dim), Linear(dim, vocab, bias=False)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, caches=None):
        x = self.embed(ids)
        caches = caches or [None] * len(self.blocks)
        new = []
        for b, c in zip(self.blocks, caches):
            x, c = b(x, c)
            new.append(c)
        return self.head(self.norm(x)), new

    @torch.no_grad()
    def generate(self, ids, max_tokens: int = 8):
        logits, caches = self.forward(torch.as_tensor(ids))
        out = []
        for _ in range(max_tokens):
            t = int(logits[-1].argmax())
            out.append(t)
            logits, caches = self.forward(torch.tensor([t]), caches)
        return out
