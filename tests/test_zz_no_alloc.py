"""The allocation-free attention entry point (``rlz_attn_decode_static``).

Some users of this library cannot allocate device memory where they call attention: the GPU
memory of their process is already fully handed out, or the host application owns the
allocator, or the call sits in a loop where cudaMalloc's device synchronisation is not
acceptable.  For them the library keeps the split-K scratch of the decode-attention kernel in a
fixed array inside the library image.  This test calls that entry point through its exported C
symbol and checks that it gives the same output as the regular entry point (which takes
caller-allocated scratch), twice in a row, because the built-in scratch is shared by all calls
and keeps the previous call's contents.

Which launches touch the built-in scratch: up to eight context splits of a head are merged inside a
thread-block cluster through shared memory and never read the scratch pointers, so the cases
below use 12 and 16 splits (partial results and arrival counters in global memory), with bf16
and int8 caches and a head size that only the scalar kernels take.  The two smaller cases keep
the cluster path covered.  With a wrong scratch address, or counters that do not return to zero,
the 12- and 16-split cases fail.

The file name makes pytest collect it last, so a run that stops at the first failure has
already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(batch, H, Hkv, d, ctx, splits, seed, q8=False):
    from realizar_b200 import ops
    torch.manual_seed(seed)
    pages_per_seq = -(-ctx // 16)
    n_pages = batch * pages_per_seq
    if q8:                      # int8 rows with a per-row scale, filled through the library's own append kernel
        kv = ops.kv_cache_alloc(1, n_pages, Hkv, d, "cuda", "q8")
        kc, vc = kv[0, 0], kv[1, 0]
        n_tok = n_pages * 16
        pos = torch.arange(n_tok, device="cuda", dtype=torch.int32) % (pages_per_seq * 16)
        rows = torch.arange(n_tok, device="cuda", dtype=torch.int32) // 16
        ops.kv_append((torch.randn(n_tok, Hkv * d, device="cuda") * 0.5).contiguous(), (torch.randn(n_tok, Hkv * d, device="cuda") * 0.5).contiguous(),
                      kc, vc, pos, rows.contiguous(), Hkv, d)
    else:
        kc = (torch.randn(n_pages, Hkv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
        vc = (torch.randn(n_pages, Hkv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    pt = torch.randperm(n_pages, device="cuda").to(torch.int32).reshape(batch, pages_per_seq).contiguous()
    qkv = torch.randn(batch, (H + 2 * Hkv) * d, device="cuda")
    pos = torch.tensor([ctx - 1 - 3 * b for b in range(batch)], device="cuda", dtype=torch.int32)
    return ops, kc, vc, pt, qkv, pos


@pytest.mark.parametrize("H,Hkv,d,ctx,splits,q8", [
    (8, 8, 80, 200, 4, False), (16, 4, 128, 333, 6, False),            # merged inside a cluster: scratch pointers unused
    (8, 8, 80, 400, 12, False), (16, 4, 128, 520, 16, False),           # merged through the built-in scratch
    (8, 2, 72, 300, 12, False), (8, 8, 64, 330, 16, True)])            # scalar kernels: odd head size, int8 cache
def test_static_entry_point_matches_regular_one_twice(cuda_device, H, Hkv, d, ctx, splits, q8):
    batch = 2
    ops, kc, vc, pt, qkv, pos = _setup(batch, H, Hkv, d, ctx, splits, seed=H + ctx, q8=q8)
    lib = ops.lib()
    fn = lib.rlz_attn_decode_static                       # the exported C symbol itself
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.rlz_attn_decode_static_strerror.restype = ctypes.c_char_p
    lib.rlz_attn_decode_static_strerror.argtypes = [ctypes.c_int]
    stream = torch.cuda.current_stream().cuda_stream

    def run(static: bool, qkv_in):
        # both paths append the new K/V row to the cache, so each gets its own copy of it
        k2, v2 = kc.clone(), vc.clone()
        out = torch.zeros(batch, H * d, device="cuda")
        partial, counters = ops.attn_decode_scratch(batch, H, splits, d, "cuda")
        p = ops.build_attn_decode_params(qkv_in, out, k2, v2, pos, pt, partial, counters, H, Hkv, d, splits, batch, d // 2 // 2 * 2, 2, 1e4,
                                         0, H * d, (H + Hkv) * d)
        assert p.kv_q8 == (1 if q8 else 0)
        if static:
            p.partial, p.counters = None, None             # ignored by the static entry point
            rc = fn(ctypes.addressof(p), stream)
            assert rc == 0, lib.rlz_attn_decode_static_strerror(rc)
        else:
            ops.attn_decode_launch(p)
        torch.cuda.synchronize()
        return out

    for call in range(2):                                   # second call sees the scratch the first one left behind
        q_in = qkv if call == 0 else qkv * 0.5 + 0.1
        want = run(False, q_in)
        got = run(True, q_in)
        err = float((got - want).abs().max() / (want.abs().max() + 1e-12))
        assert err < 5e-3, (call, err)


def test_static_entry_point_rejects_oversized_launch(cuda_device):
    ops, kc, vc, pt, qkv, pos = _setup(1, 8, 8, 64, 64, 2, seed=0)
    lib = ops.lib()
    lib.rlz_attn_decode_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.rlz_attn_decode_static_strerror.restype = ctypes.c_char_p
    lib.rlz_attn_decode_static_strerror.argtypes = [ctypes.c_int]
    out = torch.zeros(1, 8 * 64, device="cuda")
    partial, counters = ops.attn_decode_scratch(1, 8, 2, 64, "cuda")
    p = ops.build_attn_decode_params(qkv, out, kc, vc, pos, pt, partial, counters, 8, 8, 64, 2, 1, 0, 0, 1e4, 0, 8 * 64, 16 * 64)
    p.batch, p.splits = 4096, 64                           # 4096*8*64*66 floats: far beyond the built-in scratch
    rc = lib.rlz_attn_decode_static(ctypes.addressof(p), torch.cuda.current_stream().cuda_stream)
    assert rc == -10
    assert b"scratch" in lib.rlz_attn_decode_static_strerror(rc)
    torch.cuda.synchronize()
