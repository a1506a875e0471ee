"""Plain PyTorch fp32 decoder over dequantised weights: the numerical oracle.

It evaluates the same data flow as the C++ CPU engine and the GPU engine, but with dense
fp32 matmuls on fully dequantised weights and a whole-sequence causal attention, so every
fused / quantised path can be compared against it (reference parity for the data flow:
src/gguf/inference/forward/forward_cached.rs:11-398; tolerances: cosine >= 0.99 on logits).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .config import ROPE_NEOX, ModelConfig
from .weights import ModelWeights


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def apply_rope(x: torch.Tensor, positions: torch.Tensor, rope_dim: int, theta: float, rope_type: int) -> torch.Tensor:
    """x: [T, heads, head_dim]; rotates the first ``rope_dim`` dims of every head."""
    if rope_dim <= 0:
        return x
    half = rope_dim // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / rope_dim)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = x.clone()
    if rope_type == ROPE_NEOX:
        a, b = x[..., :half], x[..., half:rope_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rope_dim] = a * sin + b * cos
    else:
        a, b = x[..., 0:rope_dim:2], x[..., 1:rope_dim:2]
        out[..., 0:rope_dim:2] = a * cos - b * sin
        out[..., 1:rope_dim:2] = a * sin + b * cos
    return out


class ReferenceDecoder:
    """fp32 oracle.  ``forward(tokens)`` returns logits for every position ``[T, vocab]``."""

    def __init__(self, weights: ModelWeights, device="cpu"):
        self.cfg: ModelConfig = weights.config
        self.device = torch.device(device)
        self.w: Dict[str, torch.Tensor] = {}
        for name, t in weights.tensors.items():
            self.w[name] = torch.from_numpy(t.to_f32()).to(self.device)
        if "output.weight" not in self.w:
            self.w["output.weight"] = self.w["token_embd.weight"]

    def _norm(self, x, wname, bname):
        c = self.cfg
        w, b = self.w.get(wname), self.w.get(bname)
        if c.uses_layernorm:
            mean = x.mean(-1, keepdim=True)
            var = ((x - mean) ** 2).mean(-1, keepdim=True)
            y = (x - mean) / torch.sqrt(var + c.eps)
        else:
            y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + c.eps)
        if w is not None:
            y = y * w
        if b is not None:
            y = y + b
        return y

    def _lin(self, x, name):
        y = x @ self.w[name + ".weight"].T
        b = self.w.get(name + ".bias")
        return y + b if b is not None else y

    @torch.no_grad()
    def forward(self, tokens, collect: Optional[dict] = None) -> torch.Tensor:
        c = self.cfg
        tokens = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        T = tokens.numel()
        pos = torch.arange(T, device=self.device)
        x = self.w["token_embd.weight"][tokens]
        if "token_pos_embd.weight" in self.w:
            x = x + self.w["token_pos_embd.weight"][pos]
        mask = torch.full((T, T), float("-inf"), device=self.device).triu(1)
        group = c.num_heads // c.num_kv_heads
        for l in range(c.num_layers):
            p = f"blk.{l}."
            h = self._norm(x, p + "attn_norm.weight", p + "attn_norm.bias")
            if p + "attn_qkv.weight" in self.w:
                qkv = self._lin(h, p + "attn_qkv")
                q, k, v = qkv.split([c.q_dim, c.kv_dim, c.kv_dim], dim=-1)
            else:
                q, k, v = self._lin(h, p + "attn_q"), self._lin(h, p + "attn_k"), self._lin(h, p + "attn_v")
            q = q.reshape(T, c.num_heads, c.head_dim)
            k = k.reshape(T, c.num_kv_heads, c.head_dim)
            v = v.reshape(T, c.num_kv_heads, c.head_dim)
            if p + "attn_q_norm.weight" in self.w:
                q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + c.eps) * self.w[p + "attn_q_norm.weight"]
                k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + c.eps) * self.w[p + "attn_k_norm.weight"]
            if c.uses_rope:
                q = apply_rope(q, pos, c.rope_dim, c.rope_theta, c.rope_type)
                k = apply_rope(k, pos, c.rope_dim, c.rope_theta, c.rope_type)
            kk = k.repeat_interleave(group, dim=1)
            vv = v.repeat_interleave(group, dim=1)
            s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(c.head_dim) + mask
            a = torch.einsum("hts,shd->thd", s.softmax(-1), vv).reshape(T, c.q_dim)
            attn = self._lin(a, p + "attn_output")
            if c.parallel_residual:
                f_in = h
            else:
                x = x + attn
                f_in = self._norm(x, p + "ffn_norm.weight", p + "ffn_norm.bias")
            if c.gated_ffn:
                g = self._lin(f_in, p + "ffn_gate")
                act = torch.nn.functional.silu(g) if c.constraints.activation == "silu" else gelu_tanh(g)
                f = act * self._lin(f_in, p + "ffn_up")
            else:
                f = gelu_tanh(self._lin(f_in, p + "ffn_up"))
            f = self._lin(f, p + "ffn_down")
            x = x + attn + f if c.parallel_residual else x + f
            if collect is not None:
                collect[f"layer{l}"] = x.clone()
        x = self._norm(x, "output_norm.weight", "output_norm.bias")
        return self._lin(x, "output")

    @torch.no_grad()
    def generate_greedy(self, prompt, n_gen: int):
        toks = list(prompt)
        out = []
        for _ in range(n_gen):
            nxt = int(self.forward(toks)[-1].argmax())
            out.append(nxt)
            toks.append(nxt)
        return out
