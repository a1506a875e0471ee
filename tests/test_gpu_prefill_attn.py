"""Tensor-core flash prefill attention against a plain fp32 PyTorch restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, pos0, window):
    """q [T, H, d]; k, v [ctx, Hkv, d] (fp32).  Causal softmax attention of rows at positions pos0.."""
    T, H, d = q.shape
    ctx, Hkv, _ = k.shape
    rep = H // Hkv
    kh, vh = k.repeat_interleave(rep, 1).permute(1, 0, 2), v.repeat_interleave(rep, 1).permute(1, 0, 2)
    s = q.permute(1, 0, 2) @ kh.transpose(1, 2) / math.sqrt(d)
    qpos = torch.arange(pos0, pos0 + T, device=q.device)[:, None]
    kpos = torch.arange(ctx, device=q.device)[None, :]
    mask = kpos > qpos
    if window:
        mask = mask | (kpos <= qpos - window)
    s = s.masked_fill(mask[None], float("-inf"))
    return (torch.softmax(s, -1) @ vh).permute(1, 0, 2)


@pytest.mark.parametrize("impl", ["tc", "mma"])            # both kernels at every head size, whatever the launcher would pick
@pytest.mark.parametrize("d,H,Hkv", [(64, 8, 2), (80, 4, 4), (128, 8, 1), (96, 2, 2)])
@pytest.mark.parametrize("T,pos0,window", [(40, 0, 0), (128, 0, 0), (300, 37, 0), (200, 150, 64)])
def test_flash_prefill_matches_reference(cuda_device, d, H, Hkv, T, pos0, window, impl):
    from realizar_b200 import ops
    assert ops.attn_prefill_supported(d)
    dev = cuda_device
    g = torch.Generator(device="cpu").manual_seed(d * 1000 + T)
    ctx = pos0 + T
    n_pages = -(-ctx // 16)
    total_pages = n_pages + 5
    perm = torch.randperm(total_pages, generator=g)[:n_pages].to(torch.int32)
    k = torch.randn(ctx, Hkv, d, generator=g)
    v = torch.randn(ctx, Hkv, d, generator=g)
    q = torch.randn(T, H, d, generator=g)
    kc = torch.zeros(total_pages, Hkv, 16, d, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for p in range(ctx):
        kc[perm[p // 16], :, p % 16] = k[p].to(torch.bfloat16)
        vc[perm[p // 16], :, p % 16] = v[p].to(torch.bfloat16)
    ld = H * d + 24                                           # row pitch with padding, q section at an offset
    qkv = torch.zeros(T, ld)
    qkv[:, 8:8 + H * d] = q.reshape(T, -1)
    out = torch.full((T, H * d + 4), float("nan"), device=dev)
    ops.attn_prefill(qkv.to(dev), out, kc.to(dev), vc.to(dev), perm.to(dev), T, pos0, H, Hkv, d, q_off=8, window=window, impl=impl)
    torch.cuda.synchronize()
    assert ops.attn_prefill_error() == 0
    # the kernel sees bf16 q / k / v: give the reference the same rounded inputs
    want = _reference(q.to(torch.bfloat16).float().to(dev), k.to(torch.bfloat16).float().to(dev), v.to(torch.bfloat16).float().to(dev), pos0, window)
    got = out[:, :H * d].reshape(T, H, d)
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err < 3e-2, err                                    # P is rounded to bf16 before the PV product
    assert torch.isnan(out[:, H * d:]).all()                 # nothing written outside the head columns


def test_flash_prefill_used_by_engine_prefill(cuda_device):
    """A 200-token prompt through the engine: flash path and per-row decode-kernel path agree."""
    import numpy as np
    from realizar_b200.models.config import ModelConfig, arch_constraints
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig
    cfg = ModelConfig("llama", 512, 2, 8, 2, 64, 1024, 512, 512, 1e4, 64, 0, 1e-5, 1, 2, arch_constraints("llama"))
    w = synthetic_weights(cfg, seed=11, std=0.05)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg.vocab_size, 200)]
    res = []
    for flash in (True, False):
        eng = DecodeEngine(w, EngineConfig(max_batch=1, max_seq_len=256, greedy_only=True, prefill_chunk=128))
        assert eng.batched().flash_ok
        eng.batched().flash_ok = flash
        eng.open_slot(0, 256)
        eng.prefill(0, toks)
        res.append(eng.logits_of_last_step(0).float().cpu().numpy())
    a, b = res
    assert float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b))) > 0.999
