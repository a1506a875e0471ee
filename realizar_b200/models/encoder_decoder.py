"""Encoder-decoder transformer (T5 / Whisper style): a bidirectional encoder, a causal decoder
with cross-attention over the encoder output, T5 relative-position bias buckets, LayerNorm (or
T5's scale-only RMS norm) and a GELU / ReLU feed-forward.  PyTorch modules with an incremental
decoder cache (self-attention K/V grow, cross-attention K/V computed once).
Reference parity: ``encode`` / ``decode`` (src/gguf/inference/forward/encoder_decoder.rs:1-247,
encoder_decoder_decode.rs:1-184), ``is_encoder_decoder`` (src/gguf/config.rs:462)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass
class EncDecConfig:
    vocab_size: int = 256
    hidden_dim: int = 64
    num_heads: int = 4
    head_dim: int = 16
    ffn_dim: int = 128
    enc_layers: int = 2
    dec_layers: int = 2
    rel_buckets: int = 32
    rel_max_distance: int = 128
    use_rel_bias: bool = True          # T5; Whisper uses absolute positions instead
    max_positions: int = 512
    activation: str = "gelu"
    eps: float = 1e-6
    decoder_start_token_id: int = 0
    eos_token_id: int = 1


def relative_position_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """T5 bucketing: exact buckets for small offsets, logarithmic ones up to ``max_distance``."""
    ret = torch.zeros_like(rel)
    n = -rel
    if bidirectional:
        num_buckets //= 2
        ret = ret + (n < 0).long() * num_buckets
        n = n.abs()
    else:
        n = n.clamp(min=0)
    max_exact = num_buckets // 2
    is_small = n < max_exact
    large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact) * (num_buckets - max_exact)).long()
    large = large.clamp(max=num_buckets - 1)
    return ret + torch.where(is_small, n, large)


class _Attn(torch.nn.Module):
    def __init__(self, c: EncDecConfig, g: torch.Generator, rel_bias: bool, bidirectional: bool):
        super().__init__()
        inner = c.num_heads * c.head_dim
        p = lambda *s: torch.nn.Parameter(torch.randn(*s, generator=g) * s[-1] ** -0.5)
        self.q, self.k, self.v, self.o = p(inner, c.hidden_dim), p(inner, c.hidden_dim), p(inner, c.hidden_dim), p(c.hidden_dim, inner)
        self.c, self.bidirectional = c, bidirectional
        self.rel = torch.nn.Parameter(torch.randn(c.rel_buckets, c.num_heads, generator=g) * 0.1) if rel_bias else None

    def bias(self, q_pos: torch.Tensor, k_pos: torch.Tensor) -> Optional[torch.Tensor]:
        if self.rel is None:
            return None
        b = relative_position_bucket(k_pos[None, :] - q_pos[:, None], self.bidirectional, self.c.rel_buckets, self.c.rel_max_distance)
        return self.rel[b].permute(2, 0, 1)                      # [H, Tq, Tk]

    def attend(self, xq, k, v, q_pos, k_pos, causal: bool) -> torch.Tensor:
        c = self.c
        Tq, Tk = xq.shape[0], k.shape[0]
        q = (xq @ self.q.t()).view(Tq, c.num_heads, c.head_dim).transpose(0, 1)
        kh = k.view(Tk, c.num_heads, c.head_dim).transpose(0, 1)
        vh = v.view(Tk, c.num_heads, c.head_dim).transpose(0, 1)
        scale = 1.0 if self.rel is not None else c.head_dim ** -0.5        # T5 folds the scale into its initialisation
        s = q @ kh.transpose(1, 2) * scale
        b = self.bias(q_pos, k_pos)
        if b is not None:
            s = s + b
        if causal:
            s = s.masked_fill(k_pos[None, None, :] > q_pos[None, :, None], float("-inf"))
        return (torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(Tq, -1) @ self.o.t()


class _Norm(torch.nn.Module):
    def __init__(self, c: EncDecConfig):
        super().__init__()
        self.w = torch.nn.Parameter(torch.ones(c.hidden_dim))
        self.b = None if c.use_rel_bias else torch.nn.Parameter(torch.zeros(c.hidden_dim))
        self.eps = c.eps

    def forward(self, x):
        if self.b is None:
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.eps) * self.w
        return F.layer_norm(x, x.shape[-1:], self.w, self.b, self.eps)


class _Ffn(torch.nn.Module):
    def __init__(self, c: EncDecConfig, g):
        super().__init__()
        p = lambda *s: torch.nn.Parameter(torch.randn(*s, generator=g) * s[-1] ** -0.5)
        self.wi, self.wo, self.act = p(c.ffn_dim, c.hidden_dim), p(c.hidden_dim, c.ffn_dim), c.activation

    def forward(self, x):
        h = x @ self.wi.t()
        return (F.gelu(h) if self.act == "gelu" else F.relu(h)) @ self.wo.t()


@dataclass
class DecoderCache:
    self_k: List[torch.Tensor] = field(default_factory=list)
    self_v: List[torch.Tensor] = field(default_factory=list)
    cross_k: List[torch.Tensor] = field(default_factory=list)
    cross_v: List[torch.Tensor] = field(default_factory=list)
    length: int = 0


class EncoderDecoderModel(torch.nn.Module):
    def __init__(self, cfg: EncDecConfig, seed: int = 0):
        super().__init__()
        c, g = cfg, torch.Generator().manual_seed(seed)
        self.cfg = c
        self.embed = torch.nn.Parameter(torch.randn(c.vocab_size, c.hidden_dim, generator=g) * 0.5)
        self.pos = None if c.use_rel_bias else torch.nn.Parameter(torch.randn(c.max_positions, c.hidden_dim, generator=g) * 0.02)
        mk = torch.nn.ModuleList
        # the first layer of each stack owns the relative-position table (shared by the others, as in T5)
        self.enc_attn = mk([_Attn(c, g, c.use_rel_bias and i == 0, True) for i in range(c.enc_layers)])
        self.enc_ffn = mk([_Ffn(c, g) for _ in range(c.enc_layers)])
        self.enc_n1, self.enc_n2 = mk([_Norm(c) for _ in range(c.enc_layers)]), mk([_Norm(c) for _ in range(c.enc_layers)])
        self.dec_self = mk([_Attn(c, g, c.use_rel_bias and i == 0, False) for i in range(c.dec_layers)])
        self.dec_cross = mk([_Attn(c, g, False, True) for _ in range(c.dec_layers)])
        self.dec_ffn = mk([_Ffn(c, g) for _ in range(c.dec_layers)])
        self.dec_n1, self.dec_n2, self.dec_n3 = (mk([_Norm(c) for _ in range(c.dec_layers)]) for _ in range(3))
        self.enc_final, self.dec_final = _Norm(c), _Norm(c)

    def _emb(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        x = self.embed[ids]
        return x if self.pos is None else x + self.pos[pos]

    @torch.no_grad()
    def encode(self, ids: torch.Tensor) -> torch.Tensor:
        T = ids.shape[0]
        pos = torch.arange(T)
        x = self._emb(ids, pos)
        bias_owner = self.enc_attn[0]
        for a, f, n1, n2 in zip(self.enc_attn, self.enc_ffn, self.enc_n1, self.enc_n2):
            h = n1(x)
            a_rel, a.rel = a.rel, bias_owner.rel
            x = x + a.attend(h, h @ a.k.t(), h @ a.v.t(), pos, pos, causal=False)
            a.rel = a_rel
            x = x + f(n2(x))
        return self.enc_final(x)

    @torch.no_grad()
    def decode(self, ids: torch.Tensor, enc: torch.Tensor, cache: Optional[DecoderCache] = None) -> Tuple[torch.Tensor, DecoderCache]:
        """Decode ``ids`` (new tokens only when ``cache`` is given).  Returns logits [T, vocab]."""
        c = self.cfg
        cache = cache or DecoderCache()
        T, p0 = ids.shape[0], cache.length
        q_pos, enc_pos = torch.arange(p0, p0 + T), torch.arange(enc.shape[0])
        x = self._emb(ids, q_pos)
        first = not cache.cross_k
        owner = self.dec_self[0]
        for l, (sa, ca, f, n1, n2, n3) in enumerate(zip(self.dec_self, self.dec_cross, self.dec_ffn, self.dec_n1, self.dec_n2, self.dec_n3)):
            h = n1(x)
            k_new, v_new = h @ sa.k.t(), h @ sa.v.t()
            if len(cache.self_k) <= l:
                cache.self_k.append(k_new); cache.self_v.append(v_new)
            else:
                cache.self_k[l] = torch.cat([cache.self_k[l], k_new]); cache.self_v[l] = torch.cat([cache.self_v[l], v_new])
            sa_rel, sa.rel = sa.rel, owner.rel
            x = x + sa.attend(h, cache.self_k[l], cache.self_v[l], q_pos, torch.arange(p0 + T), causal=True)
            sa.rel = sa_rel
            if first:
                cache.cross_k.append(enc @ ca.k.t()); cache.cross_v.append(enc @ ca.v.t())
            x = x + ca.attend(n2(x), cache.cross_k[l], cache.cross_v[l], q_pos, enc_pos, causal=False)
            x = x + f(n3(x))
        cache.length = p0 + T
        x = self.dec_final(x)
        if c.use_rel_bias:
            x = x * c.hidden_dim ** -0.5              # T5 ties the output projection to the scaled embedding
        return x @ self.embed.t(), cache

    @torch.no_grad()
    def generate(self, src_ids, max_tokens: int = 16) -> List[int]:
        enc = self.encode(torch.as_tensor(src_ids))
        out, cache = [], None
        tok = self.cfg.decoder_start_token_id
        for _ in range(max_tokens):
            logits, cache = self.decode(torch.tensor([tok]), enc, cache)
            tok = int(logits[-1].argmax())
            out.append(tok)
            if tok == self.cfg.eos_token_id:
                break
        return out
