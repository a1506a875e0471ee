"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import numpy as np
import pytest
import torch

from realizar_b200 import quant
from realizar_b200.quant import QType

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-12))


def _weight(n, k, qt, seed=0, std=0.02):
    from realizar_b200 import ops
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    q = quant.quantize(w, qt)
    wd = torch.from_numpy(quant.dequantize(q, qt, (n, k)))
    return ops.upload_weight(q, qt, n, k, "cuda"), wd


FAST = [QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.Q8_0, QType.Q4_0]
GENERIC = [QType.Q4_1, QType.Q5_0, QType.Q5_1, QType.Q2_K, QType.F16, QType.BF16, QType.F32]


@pytest.mark.parametrize("qt", FAST + GENERIC)
@pytest.mark.parametrize("batch", [1, 3])
def test_gemv_matches_fp32(cuda_device, qt, batch):
    from realizar_b200 import ops
    n, k = 300, 1024
    w, wd = _weight(n, k, qt, seed=int(qt))
    x = torch.randn(batch, k, device="cuda")
    y = ops.gemv(w, x)
    ref = x.cpu() @ wd.T
    tol = 0.02 if qt in FAST else 2e-3       # int8 activations on the fast path
    assert _rel(y, ref) < tol, (qt, _rel(y, ref))


@pytest.mark.parametrize("n,k", [(37, 256), (2560, 2560), (513, 10240), (1000, 4096)])
@pytest.mark.parametrize("stream", [False, True])
def test_gemv_shapes_q4k(cuda_device, n, k, stream):
    from realizar_b200 import ops
    w, wd = _weight(n, k, QType.Q4_K, seed=n)
    x = torch.randn(1, k, device="cuda")
    assert _rel(ops.gemv(w, x, stream=stream), x.cpu() @ wd.T) < 0.02
    assert ops.device_error() == 0


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K])
@pytest.mark.parametrize("batch", [1, 2, 4])
def test_gemv_stream_kernel_matches_register_kernel(cuda_device, qt, batch):
    """The TMA-streamed kernel and the register-path kernel share prologue / epilogue semantics."""
    from realizar_b200 import ops
    n, k = 3000, 2048
    w, wd = _weight(n, k, qt, seed=21)
    x = torch.randn(batch, k, device="cuda") * 2
    g = torch.rand(k, device="cuda") + 0.5
    bias, res = torch.randn(n, device="cuda") * 0.1, torch.randn(batch, n, device="cuda")
    a = ops.gemv(w, x, bias=bias, act=ops.ACT_SILU, residual=res, norm=ops.NORM_RMS, norm_w=g, stream=True)
    b = ops.gemv(w, x, bias=bias, act=ops.ACT_SILU, residual=res, norm=ops.NORM_RMS, norm_w=g, stream=False)
    xc = x.cpu()
    h = xc / torch.sqrt((xc * xc).mean(-1, keepdim=True) + 1e-5) * g.cpu()
    ref = torch.nn.functional.silu(h @ wd.T + bias.cpu()) + res.cpu()
    assert _rel(a, ref) < 0.02 and _rel(b, ref) < 0.02 and _rel(a, b) < 5e-3
    assert ops.device_error() == 0


@pytest.mark.parametrize("norm", ["rms", "layer"])
@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_1])
def test_gemv_fused_norm_bias_act_residual(cuda_device, norm, qt):
    from realizar_b200 import ops
    n, k, B = 256, 512, 2
    w, wd = _weight(n, k, qt, seed=5)
    x = torch.randn(B, k, device="cuda") * 3 + 0.5
    g, b = torch.rand(k, device="cuda") + 0.5, torch.randn(k, device="cuda") * 0.1
    bias, res = torch.randn(n, device="cuda") * 0.1, torch.randn(B, n, device="cuda")
    y = ops.gemv(w, x, bias=bias, act=ops.ACT_GELU, residual=res, norm=ops.NORM_RMS if norm == "rms" else ops.NORM_LAYER,
                 norm_w=g, norm_b=b if norm == "layer" else None, eps=1e-5)
    xc = x.cpu()
    if norm == "rms":
        h = xc / torch.sqrt((xc * xc).mean(-1, keepdim=True) + 1e-5) * g.cpu()
    else:
        h = torch.nn.functional.layer_norm(xc, (k,), g.cpu(), b.cpu(), 1e-5)
    ref = torch.nn.functional.gelu(h @ wd.T + bias.cpu(), approximate="tanh") + res.cpu()
    assert _rel(y, ref) < 0.02


def test_gemv_swiglu_pair_and_dual_accumulate(cuda_device):
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn
    n, k, k2, B = 384, 512, 768, 2
    wg, wgd = _weight(n, k, QType.Q4_K, 1)
    wu, wud = _weight(n, k, QType.Q4_K, 2)
    x = torch.randn(B, k, device="cuda")
    y = torch.empty(B, n, device="cuda")
    p = ops.build_gemv_params([VecIn(x, k)], [MatOut([(wg, 0), (wu, 0)], combine=ops.COMBINE_SILU_MUL)], y, B)
    ops.gemv_launch(p)
    ref = torch.nn.functional.silu(x.cpu() @ wgd.T) * (x.cpu() @ wud.T)
    assert _rel(y, ref) < 0.03
    # two matrices with different inputs accumulated into the same rows (+ two biases + residual)
    w2, w2d = _weight(n, k2, QType.Q6_K, 3)
    x2 = torch.randn(B, k2, device="cuda")
    b1, b2, res = torch.randn(n, device="cuda"), torch.randn(n, device="cuda"), torch.randn(B, n, device="cuda")
    y2 = torch.empty(B, n, device="cuda")
    p = ops.build_gemv_params([VecIn(x, k), VecIn(x2, k2)], [MatOut([(wg, 0), (w2, 1)], bias=b1, bias2=b2, residual=True)], y2, B, residual=res)
    ops.gemv_launch(p)
    ref2 = x.cpu() @ wgd.T + x2.cpu() @ w2d.T + b1.cpu() + b2.cpu() + res.cpu()
    assert _rel(y2, ref2) < 0.02


def test_gemv_multi_matrix_launch(cuda_device):
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn
    k = 512
    ws = [_weight(n, k, qt, 10 + i) for i, (n, qt) in enumerate([(128, QType.Q4_K), (64, QType.Q4_K), (64, QType.Q6_K), (200, QType.Q5_K)])]
    x = torch.randn(1, k, device="cuda")
    total = sum(w.n for w, _ in ws)
    y = torch.zeros(1, total, device="cuda")
    mats, off = [], 0
    for w, _ in ws:
        mats.append(MatOut([(w, 0)], out_off=off))
        off += w.n
    ops.gemv_launch(ops.build_gemv_params([VecIn(x, k)], mats, y, 1))
    ref = torch.cat([x.cpu() @ wd.T for _, wd in ws], dim=-1)
    assert _rel(y, ref) < 0.02


def _launch_on(p, slab):
    from realizar_b200 import ops
    p._slab = slab
    ops.gemv_launch(p)


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K])
@pytest.mark.parametrize("batch", [1, 2, 4])
@pytest.mark.parametrize("n,k,ctas", [(3000, 2048, 296), (61, 2560, 1), (700, 10240, 148), (9, 256, 1)])
def test_gemv_slab_kernel_matches_register_kernel(cuda_device, qt, batch, n, k, ctas):
    """The copy-engine-fed kernel against the register-path kernel and an fp32 reference (fused norm, bias, act, residual)."""
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn
    w, wd = _weight(n, k, qt, seed=21 + n)
    x = torch.randn(batch, k, device="cuda") * 2 + 0.3
    g, gb = torch.rand(k, device="cuda") + 0.5, torch.randn(k, device="cuda") * 0.1
    bias, res = torch.randn(n, device="cuda") * 0.1, torch.randn(batch, n, device="cuda")
    outs = []
    for slab in (True, False):
        y = torch.zeros(batch, n, device="cuda")
        p = ops.build_gemv_params([VecIn(x, k, norm=ops.NORM_LAYER, norm_w=g, norm_b=gb, eps=1e-5)], [MatOut([(w, 0)], bias=bias, act=ops.ACT_SILU, residual=True)],
                                  y, batch, residual=res, target_ctas=ctas)
        if slab and not ops.slab_eligible(p):
            assert batch * k > 16384           # only activations too large for half an SM's shared memory are turned away
            return
        _launch_on(p, slab)
        outs.append(y)
    h = torch.nn.functional.layer_norm(x.cpu(), (k,), g.cpu(), gb.cpu(), 1e-5)
    ref = torch.nn.functional.silu(h @ wd.T + bias.cpu()) + res.cpu()
    assert _rel(outs[0], ref) < 0.02 and _rel(outs[1], ref) < 0.02 and _rel(outs[0], outs[1]) < 5e-3
    assert ops.device_error() == 0


def test_gemv_slab_two_segments_multi_matrix_and_handoff(cuda_device):
    """Two accumulated segments with different inputs and block types, a four-matrix launch, and the int8 hand-off:
    the producer's quantised output block is consumed by the next launch without re-quantising."""
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn
    n, k, k2 = 2560, 2560, 10240
    wo, wod = _weight(n, k, QType.Q4_K, 1)
    wdn, wdd = _weight(n, k2, QType.Q6_K, 2)
    x, x2 = torch.randn(1, k, device="cuda"), torch.randn(1, k2, device="cuda")
    b1, b2, res = torch.randn(n, device="cuda"), torch.randn(n, device="cuda"), torch.randn(1, n, device="cuda")
    y = torch.empty(1, n, device="cuda")
    p = ops.build_gemv_params([VecIn(x, k), VecIn(x2, k2)], [MatOut([(wo, 0), (wdn, 1)], bias=b1, bias2=b2, residual=True)], y, 1, residual=res,
                              target_ctas=296)
    assert ops.slab_eligible(p)
    _launch_on(p, True)
    ref = x.cpu() @ wod.T + x2.cpu() @ wdd.T + b1.cpu() + b2.cpu() + res.cpu()
    assert _rel(y, ref) < 0.02
    # producer (register or slab kernel) writes gelu(W x) both as fp32 and as the int8 block; the consumer stages the block
    wu, wud = _weight(k2, k, QType.Q4_K, 3)
    for producer_slab in (True, False):
        act = torch.zeros(1, k2, device="cuda")
        act_q = torch.zeros(ops.act_block_bytes(k2), device="cuda", dtype=torch.uint8)
        up = MatOut([(wu, 0)], act=ops.ACT_GELU)
        up.q_out, up.q_out_k, up.q_out_col0 = act_q, k2, 0
        _launch_on(ops.build_gemv_params([VecIn(x, k)], [up], act, 1, target_ctas=296), producer_slab)
        y_pre, y_f32 = torch.empty(1, n, device="cuda"), torch.empty(1, n, device="cuda")
        _launch_on(ops.build_gemv_params([VecIn(act, k2, pre=act_q)], [MatOut([(wdn, 0)])], y_pre, 1, target_ctas=296), True)
        _launch_on(ops.build_gemv_params([VecIn(act, k2)], [MatOut([(wdn, 0)])], y_f32, 1, target_ctas=296), True)
        ref = torch.nn.functional.gelu(x.cpu() @ wud.T, approximate="tanh") @ wdd.T
        assert _rel(y_pre, ref) < 0.03 and _rel(y_pre, y_f32) < 1e-5
    # four matrices of three block types sharing one input
    ws = [_weight(nn, k, qt, 10 + i) for i, (nn, qt) in enumerate([(2560, QType.Q4_K), (640, QType.Q4_K), (640, QType.Q6_K), (3000, QType.Q5_K)])]
    total = sum(w.n for w, _ in ws)
    ym = torch.zeros(1, total, device="cuda")
    mats, off = [], 0
    for w, _ in ws:
        mats.append(MatOut([(w, 0)], out_off=off))
        off += w.n
    p = ops.build_gemv_params([VecIn(x, k)], mats, ym, 1, target_ctas=296)
    assert ops.slab_eligible(p)
    _launch_on(p, True)
    assert _rel(ym, torch.cat([x.cpu() @ wd.T for _, wd in ws], dim=-1)) < 0.02
    assert ops.device_error() == 0


def _ref_attention(q, kc, vc, scale):
    # q [H, d]; kc/vc [T, Hkv, d]
    H, d = q.shape
    Hkv = kc.shape[1]
    g = H // Hkv
    kk, vv = kc.repeat_interleave(g, dim=1), vc.repeat_interleave(g, dim=1)
    s = torch.einsum("hd,thd->ht", q, kk) * scale
    return torch.einsum("ht,thd->hd", s.softmax(-1), vv)


@pytest.mark.parametrize("H,Hkv,d,rope_dim,rope_type", [(8, 8, 80, 32, 2), (8, 2, 128, 128, 0), (14, 2, 64, 64, 2), (16, 2, 128, 128, 0), (4, 4, 64, 0, 0)])
@pytest.mark.parametrize("ctx", [1, 17, 300])
def test_attn_decode_matches_reference(cuda_device, H, Hkv, d, rope_dim, rope_type, ctx):
    from realizar_b200 import ops
    from realizar_b200.models.reference import apply_rope
    torch.manual_seed(ctx + H)
    B, splits, pages_per_seq = 2, 4, 32
    n_pages = B * pages_per_seq
    kc = torch.zeros(n_pages, Hkv, 16, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    page_table = torch.arange(n_pages, device="cuda", dtype=torch.int32).reshape(B, pages_per_seq).flip(1).contiguous()
    lens = [ctx, max(1, ctx // 2)]
    hist_k = [torch.randn(L - 1, Hkv, d) for L in lens]
    hist_v = [torch.randn(L - 1, Hkv, d) for L in lens]
    for b in range(B):          # history is stored already rotated, as the kernel would have written it
        for t in range(lens[b] - 1):
            pg, slot = int(page_table[b, t // 16]), t % 16
            kr = apply_rope(hist_k[b][t:t + 1], torch.tensor([t]), rope_dim, 10000.0, rope_type)[0]
            kc[pg, :, slot] = kr.to(torch.bfloat16).cuda()
            vc[pg, :, slot] = hist_v[b][t].to(torch.bfloat16).cuda()
    qkv = torch.randn(B, (H + 2 * Hkv) * d, device="cuda")
    positions = torch.tensor([L - 1 for L in lens], device="cuda", dtype=torch.int32)
    out = torch.zeros(B, H * d, device="cuda")
    partial, counters = ops.attn_decode_scratch(B, H, splits, d, "cuda")
    p = ops.build_attn_decode_params(qkv, out, kc, vc, positions, page_table, partial, counters, H, Hkv, d, splits, B, rope_dim, rope_type,
                                     10000.0, 0, H * d, (H + Hkv) * d)
    for _ in range(2):          # second launch checks the self-cleaning counters
        ops.attn_decode_launch(p)
    torch.cuda.synchronize()
    assert int(counters.abs().sum()) == 0
    for b in range(B):
        L = lens[b]
        row = qkv[b].cpu()
        q = row[: H * d].reshape(1, H, d)
        kn = row[H * d:(H + Hkv) * d].reshape(1, Hkv, d)
        vn = row[(H + Hkv) * d:].reshape(1, Hkv, d)
        pos = torch.tensor([L - 1])
        q = apply_rope(q, pos, rope_dim, 10000.0, rope_type)[0]
        kn = apply_rope(kn, pos, rope_dim, 10000.0, rope_type)
        kh = apply_rope(hist_k[b], torch.arange(L - 1), rope_dim, 10000.0, rope_type) if L > 1 else hist_k[b]
        k_all = torch.cat([kh, kn]).to(torch.bfloat16).float()
        v_all = torch.cat([hist_v[b], vn]).to(torch.bfloat16).float()
        ref = _ref_attention(q, k_all, v_all, d ** -0.5).reshape(-1)
        assert _rel(out[b], ref) < 5e-3, (b, _rel(out[b], ref))
        # the new row was appended to the cache
        pg, slot = int(page_table[b, (L - 1) // 16]), (L - 1) % 16
        assert _rel(kc[pg, :, slot].float(), kn[0].to(torch.bfloat16).float()) < 1e-2


@pytest.mark.parametrize("H,Hkv,d,B", [(32, 8, 128, 80), (16, 16, 80, 40), (8, 1, 64, 5), (12, 4, 96, 6)])
def test_attn_decode_streamed_pages_large_batch(cuda_device, H, Hkv, d, B):
    """Launches that fill the GPU several times over take K/V pages through a bulk-copy ring in shared memory (grouped heads by
    default; RLZ_ATT_MODE=2 / 3 force the streamed / tensor-core mode for every shape): sequences of different lengths, one
    split and two, partial head groups."""
    from realizar_b200 import ops
    torch.manual_seed(5)
    pages_per_seq = 8
    n_pages = B * pages_per_seq
    kc = (torch.randn(n_pages, Hkv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(n_pages, Hkv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    page_table = torch.randperm(n_pages, device="cuda").to(torch.int32).reshape(B, pages_per_seq).contiguous()
    lens = torch.randint(1, pages_per_seq * 16, (B,))
    lens[0], lens[1], lens[2], lens[3] = 1, 16, 17, pages_per_seq * 16
    for splits in (1, 2):
        k0, v0 = kc.clone(), vc.clone()
        qkv = torch.randn(B, (H + 2 * Hkv) * d, device="cuda")
        positions = (lens - 1).to(torch.int32).cuda()
        out = torch.zeros(B, H * d, device="cuda")
        partial, counters = ops.attn_decode_scratch(B, H, splits, d, "cuda")
        ops.attn_decode_launch(ops.build_attn_decode_params(qkv, out, k0, v0, positions, page_table, partial, counters, H, Hkv, d, splits, B, 0, 0,
                                                            1e4, 0, H * d, (H + Hkv) * d))
        torch.cuda.synchronize()
        assert ops.lib().rlz_attn_decode_error(1) == 0
        for b in (0, 1, 2, 3, B - 1):
            L = int(lens[b])
            pages = page_table[b, : (L + 15) // 16].long()
            k_all = kc[pages].permute(0, 2, 1, 3).reshape(-1, Hkv, d)[:L].float().clone()      # [tokens, Hkv, d]
            v_all = vc[pages].permute(0, 2, 1, 3).reshape(-1, Hkv, d)[:L].float().clone()
            row = qkv[b]
            k_all[L - 1] = row[H * d:(H + Hkv) * d].reshape(Hkv, d).to(torch.bfloat16).float()
            v_all[L - 1] = row[(H + Hkv) * d:].reshape(Hkv, d).to(torch.bfloat16).float()
            ref = _ref_attention(row[: H * d].reshape(H, d).cpu(), k_all.cpu(), v_all.cpu(), d ** -0.5).reshape(-1)
            assert _rel(out[b], ref) < 5e-3, (splits, b, L, _rel(out[b], ref))


def test_attn_decode_inactive_slot_and_qk_norm(cuda_device):
    from realizar_b200 import ops
    H, Hkv, d, B, splits = 4, 2, 64, 2, 2
    kc = torch.zeros(8, Hkv, 16, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pt = torch.arange(8, device="cuda", dtype=torch.int32).reshape(B, 4)
    qkv = torch.randn(B, (H + 2 * Hkv) * d, device="cuda")
    out = torch.full((B, H * d), 7.0, device="cuda")
    positions = torch.tensor([0, -1], device="cuda", dtype=torch.int32)
    partial, counters = ops.attn_decode_scratch(B, H, splits, d, "cuda")
    qn, kn = torch.rand(d, device="cuda") + 0.5, torch.rand(d, device="cuda") + 0.5
    ops.attn_decode_launch(ops.build_attn_decode_params(qkv, out, kc, vc, positions, pt, partial, counters, H, Hkv, d, splits, B, 0, 0, 1e4,
                                                        0, H * d, (H + Hkv) * d, qn, kn, 1e-6))
    torch.cuda.synchronize()
    assert torch.all(out[1] == 7.0)                 # idle slot untouched
    v_new = qkv[0, (H + Hkv) * d:].reshape(Hkv, d).to(torch.bfloat16).float()
    ref = v_new.repeat_interleave(H // Hkv, dim=0).reshape(-1)      # single token: output = v
    assert _rel(out[0], ref) < 1e-2
    k_new = qkv[0, H * d:(H + Hkv) * d].reshape(Hkv, d).cpu()
    k_ref = k_new / torch.sqrt((k_new * k_new).mean(-1, keepdim=True) + 1e-6) * kn.cpu()
    assert _rel(kc[0, :, 0].float(), k_ref) < 1e-2


def test_embed_norm_rope_elementwise(cuda_device):
    from realizar_b200 import ops
    from realizar_b200.models.reference import apply_rope
    rng = np.random.default_rng(0)
    V, Hd = 64, 512
    for qt in (QType.Q4_K, QType.Q8_0, QType.F32, QType.Q5_0):
        w = (rng.standard_normal((V, Hd)) * 0.05).astype(np.float32)
        q = quant.quantize(w, qt)
        table = torch.from_numpy(q).cuda()
        toks = torch.tensor([3, 63, -1, 0], device="cuda", dtype=torch.int32)
        out = torch.empty(4, Hd, device="cuda")
        ops.embed(table, qt, quant.row_bytes(qt, Hd), Hd, V, toks, out)
        ref = torch.from_numpy(quant.dequantize(q, qt, (V, Hd)))
        assert torch.allclose(out[0].cpu(), ref[3], atol=1e-6) and torch.allclose(out[1].cpu(), ref[63], atol=1e-6)
        assert float(out[2].abs().max()) == 0.0
    x = torch.randn(5, 320, device="cuda") * 2 + 1
    g, b = torch.rand(320, device="cuda"), torch.randn(320, device="cuda")
    assert _rel(ops.norm(x, g, b, ops.NORM_LAYER, 1e-5), torch.nn.functional.layer_norm(x.cpu(), (320,), g.cpu(), b.cpu(), 1e-5)) < 1e-5
    xr = x.cpu()
    assert _rel(ops.norm(x, g, None, ops.NORM_RMS, 1e-6), xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + 1e-6) * g.cpu()) < 1e-5
    for rope_type, rd in ((0, 64), (2, 32), (2, 80)):
        t = torch.randn(6, 4 * 80, device="cuda")
        pos = torch.tensor([0, 1, 5, 100, 2047, 7], device="cuda", dtype=torch.int32)
        ref = apply_rope(t.cpu().reshape(6, 4, 80), pos.cpu(), rd, 1e4, rope_type).reshape(6, -1)
        ops.rope_(t, pos, 4, 80, rd, rope_type, 1e4)
        assert _rel(t, ref) < 1e-4
    a, bb = torch.randn(7, 100, device="cuda"), torch.randn(7, 100, device="cuda")
    y = ops.elementwise(a, bb, act=ops.ACT_SILU)
    assert _rel(y, torch.nn.functional.silu(a.cpu()) * bb.cpu()) < 1e-5


def test_argmax_and_sampling(cuda_device):
    from realizar_b200 import ops
    torch.manual_seed(0)
    B, V = 3, 50257
    logits = torch.randn(B, V, device="cuda")
    logits[1, 777] = 50.0
    am = ops.argmax(logits)
    assert am.cpu().tolist() == logits.argmax(-1).cpu().tolist()
    temp = torch.tensor([0.0, 1.0, 0.8], device="cuda")
    top_k = torch.tensor([0, 40, 5], device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0], device="cuda")
    u = torch.tensor([0.3, 0.5, 0.999], device="cuda")
    out = ops.sample(logits, temp, top_k, top_p, u).cpu().tolist()
    assert out[0] == int(logits[0].argmax())            # temperature 0 -> greedy
    assert out[1] == 777                                # dominant token inside the nucleus
    top5 = logits[2].topk(5).indices.cpu().tolist()
    assert out[2] in top5
    # distribution check: top-k=4 sampling frequencies follow the softmax over the top 4
    row = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0, -3.0] + [-20.0] * 58], device="cuda")
    n = 4000
    us = torch.rand(n, device="cuda")
    counts = torch.zeros(64)
    big = row.repeat(n, 1).contiguous()
    o = ops.sample(big, torch.ones(n, device="cuda"), torch.full((n,), 4, device="cuda", dtype=torch.int32), torch.ones(n, device="cuda"), us)
    for t in o.cpu().tolist():
        counts[t] += 1
    assert counts[4:].sum() == 0
    expect = torch.softmax(row[0, :4].cpu(), -1)
    assert float((counts[:4] / n - expect).abs().max()) < 0.03
    # penalties
    lg = torch.zeros(1, 16, device="cuda"); lg[0, 3] = 2.0; lg[0, 5] = -2.0
    hist = torch.tensor([[3, 5, 3, -1]], device="cuda", dtype=torch.int32)
    ops.penalties_(lg, hist, torch.tensor([2.0], device="cuda"), torch.tensor([0.5], device="cuda"), torch.tensor([0.25], device="cuda"))
    assert abs(float(lg[0, 3]) - (1.0 - 0.5 - 0.5)) < 1e-6 and abs(float(lg[0, 5]) - (-4.0 - 0.5 - 0.25)) < 1e-6


def test_argmax_sliced_rows(cuda_device):
    """Wide vocabularies split each row over several CTAs; ties resolve to the smallest index; repeat launches reuse the scratch."""
    from realizar_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    for batch, vocab in ((1, 51200), (3, 151936), (70, 32000), (2, 16384)):
        logits = torch.randn(batch, vocab + 5, device="cuda", generator=g)[:, :vocab]      # row pitch larger than the vocabulary
        logits[0, 777] = logits[0, vocab - 3] = 50.0                                        # a tie: the smaller index wins
        val = torch.empty(batch, device="cuda")
        for _ in range(3):
            am = ops.argmax(logits, out_val=val, index_offset=11, vocab=vocab)
            assert (am.cpu() - 11).tolist() == logits.argmax(-1).cpu().tolist() or (am.cpu()[0] - 11 == 777 and (am.cpu()[1:] - 11).tolist() == logits[1:].argmax(-1).cpu().tolist())
            assert int(am[0]) - 11 == 777
            assert torch.allclose(val, logits.max(-1).values)
    neg = -torch.rand(1, 20000, device="cuda") - 1.0                                       # all-negative rows decode correctly too
    v = torch.empty(1, device="cuda")
    assert int(ops.argmax(neg, out_val=v)) == int(neg.argmax()) and torch.allclose(v, neg.max(-1).values)


@pytest.mark.parametrize("H,Hkv,d,splits", [(8, 8, 80, 4), (14, 2, 64, 2), (16, 2, 128, 1)])
def test_attn_decode_int8_kv(cuda_device, H, Hkv, d, splits):
    """int8 cache rows (codes + per-row scale): the kernel matches fp32 attention over the dequantised rows,
    and the row it appends dequantises back to the new k / v within one quantisation step."""
    from realizar_b200 import ops
    torch.manual_seed(H + d)
    B, pages_per_seq, ctx = 2, 8, 45
    n_pages = B * pages_per_seq
    kv = ops.kv_cache_alloc(1, n_pages, Hkv, d, "cuda", "q8")
    kc, vc = kv[0, 0], kv[1, 0]
    page_table = torch.arange(n_pages, device="cuda", dtype=torch.int32).reshape(B, pages_per_seq).flip(1).contiguous()
    lens = [ctx, 20]
    hist_k = [torch.randn(L - 1, Hkv, d, device="cuda") for L in lens]
    hist_v = [torch.randn(L - 1, Hkv, d, device="cuda") for L in lens]
    for b in range(B):          # history goes in through the append kernel (no RoPE in this test)
        L = lens[b] - 1
        pos = torch.arange(L, device="cuda", dtype=torch.int32)
        rows = page_table[b, (pos // 16).long()].contiguous()
        ops.kv_append(hist_k[b].reshape(L, -1).contiguous(), hist_v[b].reshape(L, -1).contiguous(), kc, vc, pos, rows, Hkv, d)
    qkv = torch.randn(B, (H + 2 * Hkv) * d, device="cuda")
    positions = torch.tensor([L - 1 for L in lens], device="cuda", dtype=torch.int32)
    out = torch.zeros(B, H * d, device="cuda")
    partial, counters = ops.attn_decode_scratch(B, H, splits, d, "cuda")
    p = ops.build_attn_decode_params(qkv, out, kc, vc, positions, page_table, partial, counters, H, Hkv, d, splits, B, 0, 0, 10000.0, 0, H * d, (H + Hkv) * d)
    assert p.kv_q8 == 1
    ops.attn_decode_launch(p)
    torch.cuda.synchronize()
    for b in range(B):
        L = lens[b]
        pages = page_table[b, : (L + 15) // 16].long()
        k_all = ops.kv_rows_to_float(kc[pages], d).permute(0, 2, 1, 3).reshape(-1, Hkv, d)[:L]      # [tokens, Hkv, d]
        v_all = ops.kv_rows_to_float(vc[pages], d).permute(0, 2, 1, 3).reshape(-1, Hkv, d)[:L]
        row = qkv[b]
        kn, vn = row[H * d:(H + Hkv) * d].reshape(Hkv, d), row[(H + Hkv) * d:].reshape(Hkv, d)
        step = kn.abs().amax(-1, keepdim=True) / 127
        assert float((k_all[L - 1] - kn).abs().max()) <= float(step.max()) * 0.51 + 1e-6      # appended row: within half a step
        assert float((k_all[: L - 1] - hist_k[b]).abs().max()) <= float(hist_k[b].abs().amax(-1).max()) / 127 * 0.51 + 1e-6
        ref = _ref_attention(row[: H * d].reshape(H, d).cpu(), k_all.cpu(), v_all.cpu(), d ** -0.5).reshape(-1)
        assert _rel(out[b], ref) < 5e-3, (b, _rel(out[b], ref))


@pytest.mark.parametrize("n", [2560, 4096, 72, 8192, 9000, 1001])
@pytest.mark.parametrize("norm", ["layer", "rms"])
def test_norm_bf16_vector_and_scalar_variants(cuda_device, n, norm):
    """Rows that fit the register-resident 16-byte-vector kernel (n % 4 == 0, n <= 8192), longer rows and odd lengths
    (scalar kernel), strided inputs: against an fp32 PyTorch computation rounded to bf16."""
    from realizar_b200 import ops
    torch.manual_seed(n)
    T = 37
    xfull = torch.randn(T, n + 8, device="cuda") * 3 + 0.5
    x = xfull[:, :n] if n % 4 == 0 else xfull[:, 1:n + 1]          # odd sizes also start off the 16-byte grid
    w, b = torch.rand(n, device="cuda") + 0.5, torch.randn(n, device="cuda") * 0.1
    out = torch.empty(T, n, device="cuda", dtype=torch.bfloat16)
    if norm == "layer":
        ops.norm_bf16(x, out, w, b, ops.NORM_LAYER, 1e-5)
        ref = torch.nn.functional.layer_norm(x.double(), (n,), w.double(), b.double(), 1e-5)
    else:
        ops.norm_bf16(x, out, w, None, ops.NORM_RMS, 1e-5)
        ref = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    torch.cuda.synchronize()
    err = (out.double() - ref).abs() / (ref.abs() + 1.0)
    assert float(err.max()) < 6e-3, float(err.max())


@pytest.mark.parametrize("cols,act,gated", [(10240, "gelu", False), (1024, "silu", True), (1002, "silu", True), (36, "gelu", False)])
def test_swiglu_and_to_bf16_vector_and_scalar_variants(cuda_device, cols, act, gated):
    from realizar_b200 import ops
    torch.manual_seed(cols)
    T = 19
    gate, up = torch.randn(T, cols, device="cuda") * 2, torch.randn(T, cols, device="cuda")
    out = torch.empty(T, cols, device="cuda", dtype=torch.bfloat16)
    ops.swiglu_bf16(gate, up if gated else None, out, ops.ACT_SILU if act == "silu" else ops.ACT_GELU)
    g = gate.double()
    ref = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    if gated:
        ref = ref * up.double()
    assert float(((out.double() - ref).abs() / (ref.abs() + 1.0)).max()) < 6e-3
    conv = ops.to_bf16(gate)
    assert torch.equal(conv, gate.to(torch.bfloat16))
    view = gate[:, 4:cols - 4] if cols % 4 == 0 else gate[:, 1:]
    assert torch.equal(ops.to_bf16(view), view.to(torch.bfloat16))


@pytest.mark.parametrize("world,K", [(2, 1024), (4, 1024), (8, 256)])
def test_sharded_sampling_emulated_ranks_match_full_row_sampler(cuda_device, world, K):
    """Vocabulary-sharded sampling: every emulated rank pushes the candidates of its slice (one launch per rank, none of them
    waits), then every rank merges; each must pick exactly what the one-kernel sampler picks on the whole row."""
    import ctypes
    from realizar_b200 import ops
    from realizar_b200.ops import _signatures as S
    torch.manual_seed(world)
    B, V = 6, 5003
    vl = -(-V // world)
    logits = torch.randn(B, V, device="cuda") * 3
    temperature = torch.tensor([0.7, 0.0, 1.0, 0.9, 1.3, 0.8], device="cuda")
    top_k = torch.tensor([40, 0, 1, 0, 2000, 200], device="cuda", dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 1.0, 0.5, 1.0, 0.95], device="cuda")
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.01, 0.0], device="cuda")
    for trial in range(3):
        uniform = torch.rand(B, device="cuda")
        want = ops.sample(logits, temperature, top_k, top_p, uniform, min_p)
        if K < 1024:                                        # a narrower exchange caps every row's candidate count at K
            want = ops.sample(logits, temperature, torch.where((top_k <= 0) | (top_k > K), torch.full_like(top_k, K), top_k), top_p, uniform, min_p)
        inbox = [torch.zeros(2 * world * B * K, 2, device="cuda", dtype=torch.int32) for _ in range(world)]
        flags = [torch.zeros(2 * world * B, device="cuda", dtype=torch.int32) for _ in range(world)]
        epoch = torch.full((1,), 5 + trial, device="cuda", dtype=torch.int32)
        status = torch.zeros(1, device="cuda", dtype=torch.int32)
        outs = [torch.full((B,), -1, device="cuda", dtype=torch.int32) for _ in range(world)]
        descs, sps = [], []
        for r in range(world):
            c = S.ShardSample()
            for q in range(world):
                c.inbox[q], c.flags[q] = inbox[q].data_ptr(), flags[q].data_ptr()
            c.epoch, c.status, c.spin_limit = epoch.data_ptr(), status.data_ptr(), 1000
            c.rank, c.world, c.batch_cap, c.K, c.index_offset = r, world, B, K, r * vl
            n_local = max(0, min(V, (r + 1) * vl) - r * vl)
            sp = ops.build_sample_params(logits[:, r * vl:], temperature, top_k, top_p, uniform, outs[r], min_p, vocab=n_local)
            descs.append(c); sps.append(sp)
        for r in range(world):
            ops.check(ops.lib().rlz_sample_push(ctypes.byref(sps[r]), ctypes.byref(descs[r]), ops.stream_ptr()), "push")
        for r in range(world):
            ops.check(ops.lib().rlz_sample_merge(ctypes.byref(sps[r]), ctypes.byref(descs[r]), ops.stream_ptr()), "merge")
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for r in range(world):
            assert torch.equal(outs[r], want), (r, outs[r].tolist(), want.tolist())
    # a list that never arrives: the wait runs out, the status word says so, the draw uses what is there
    flags[0].zero_()
    ops.check(ops.lib().rlz_sample_merge(ctypes.byref(sps[0]), ctypes.byref(descs[0]), ops.stream_ptr()), "merge")
    torch.cuda.synchronize()
    assert int(status.item()) == 2006
