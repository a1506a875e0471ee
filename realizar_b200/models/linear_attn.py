"""Gated DeltaNet ("linear attention") layer state and recurrence, as used by hybrid-attention
models: per head a matrix state ``S`` (d_k × d_v) updated by the gated delta rule

    S_t = exp(g_t) · S_{t-1} + k_t ⊗ δ_t,   δ_t = β_t (v_t − S_{t-1}ᵀ k_t · exp(g_t)),   o_t = S_tᵀ q_t

preceded by a depth-wise causal conv1d over the last ``conv_k`` inputs and followed by a gated
RMSNorm.  Reference parity: ``LinearAttnState`` and the recurrence in
src/gpu/scheduler/linear_attn.rs:1-60 ff., src/gpu/scheduler/types.rs:79-116."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass
class LinearAttnConfig:
    num_heads: int
    key_dim: int
    value_dim: int
    conv_kernel: int = 4
    eps: float = 1e-6


class LinearAttnState:
    """Recurrent state of one layer for one sequence: ``S`` [H, d_k, d_v] and the conv window."""

    def __init__(self, cfg: LinearAttnConfig, conv_channels: int, device="cpu", dtype=torch.float32):
        self.cfg = cfg
        self.S = torch.zeros(cfg.num_heads, cfg.key_dim, cfg.value_dim, device=device, dtype=dtype)
        self.conv = torch.zeros(conv_channels, cfg.conv_kernel - 1, device=device, dtype=dtype)

    def reset(self) -> None:
        self.S.zero_()
        self.conv.zero_()

    def clone(self) -> "LinearAttnState":
        c = LinearAttnState.__new__(LinearAttnState)
        c.cfg, c.S, c.conv = self.cfg, self.S.clone(), self.conv.clone()
        return c


def causal_conv1d_step(x: torch.Tensor, state: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depth-wise causal convolution for one new time step.  ``x`` [C], ``state`` [C, K-1]
    (oldest first, updated in place), ``weight`` [C, K]."""
    window = torch.cat([state, x.unsqueeze(1)], dim=1)
    y = (window * weight).sum(1)
    state.copy_(window[:, 1:])
    return F.silu(y + bias if bias is not None else y)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta_step(S: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """One token.  ``S`` [H, dk, dv] updated in place; ``q``,``k`` [H, dk]; ``v`` [H, dv]; ``g`` (log decay ≤ 0), ``beta`` [H]."""
    S.mul_(torch.exp(g)[:, None, None])
    pred = torch.einsum("hkv,hk->hv", S, k)
    delta = beta[:, None] * (v - pred)
    S.add_(k[:, :, None] * delta[:, None, :])
    return torch.einsum("hkv,hk->hv", S, q)


def gated_delta_chunk(S: torch.Tensor, q, k, v, g, beta) -> torch.Tensor:
    """A run of T tokens (prefill): sequential over time, batched over heads."""
    return torch.stack([gated_delta_step(S, q[t], k[t], v[t], g[t], beta[t]) for t in range(q.shape[0])])


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    n = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight
    return n * F.silu(gate)


class GatedDeltaNetLayer(torch.nn.Module):
    """Projection → conv → recurrence → gated norm → output projection for a token stream."""

    def __init__(self, hidden: int, cfg: LinearAttnConfig, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        H, dk, dv = cfg.num_heads, cfg.key_dim, cfg.value_dim
        self.qkv_dim = H * (2 * dk + dv)
        g = torch.Generator().manual_seed(seed)
        p = lambda *s: torch.nn.Parameter(torch.randn(*s, generator=g) * s[-1] ** -0.5)
        self.in_proj = p(self.qkv_dim, hidden)
        self.z_proj = p(H * dv, hidden)
        self.ba_proj = p(2 * H, hidden)
        self.conv_w = p(self.qkv_dim, cfg.conv_kernel)
        self.A_log = torch.nn.Parameter(torch.zeros(H))
        self.dt_bias = torch.nn.Parameter(torch.zeros(H))
        self.norm_w = torch.nn.Parameter(torch.ones(dv))
        self.out_proj = p(hidden, H * dv)

    def new_state(self) -> LinearAttnState:
        return LinearAttnState(self.cfg, self.qkv_dim, self.in_proj.device, self.in_proj.dtype)

    @torch.no_grad()
    def step(self, x: torch.Tensor, st: LinearAttnState) -> torch.Tensor:
        c = self.cfg
        H, dk, dv = c.num_heads, c.key_dim, c.value_dim
        mixed = causal_conv1d_step(self.in_proj @ x, st.conv, self.conv_w)
        q, k, v = mixed.split([H * dk, H * dk, H * dv])
        q, k, v = l2norm(q.view(H, dk)) * dk ** -0.5, l2norm(k.view(H, dk)), v.view(H, dv)
        b, a = (self.ba_proj @ x).split([H, H])
        beta = torch.sigmoid(b)
        g = -torch.exp(self.A_log) * F.softplus(a + self.dt_bias)
        o = gated_delta_step(st.S, q, k, v, g, beta)
        o = gated_rmsnorm(o, (self.z_proj @ x).view(H, dv), self.norm_w, c.eps)
        return self.out_proj @ o.reshape(-1)

    @torch.no_grad()
    def forward(self, xs: torch.Tensor, st: Optional[LinearAttnState] = None) -> Tuple[torch.Tensor, LinearAttnState]:
        st = st or self.new_state()
        return torch.stack([self.step(x, st) for x in xs]), st
