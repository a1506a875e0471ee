"""tcgen05 dequant-GEMM against an fp32 reference on dequantised weights and bf16-rounded inputs."""
import numpy as np
import pytest
import torch

from realizar_b200 import quant
from realizar_b200.quant import QType

pytestmark = pytest.mark.gpu


def _weight(n, k, qt, seed):
    from realizar_b200 import ops
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.05).astype(np.float32)
    q = quant.quantize(w, qt)
    return ops.upload_weight(q, qt, n, k, "cuda"), torch.from_numpy(quant.dequantize(q, qt, (n, k)))


@pytest.mark.parametrize("qt", [QType.Q4_0, QType.Q4_1, QType.Q5_0, QType.Q5_1, QType.Q8_0])
@pytest.mark.parametrize("m,n,k,splitk", [(5, 128, 64, 1), (64, 200, 576, 1), (130, 384, 1024, 1), (300, 250, 2560, 1), (20, 256, 2048, 4)])
def test_gemm_32_weight_block_types(cuda_device, qt, m, n, k, splitk):
    """The 32-weight block types (planar Q4_0 / Q8_0 rows, interleaved Q4_1 / Q5_0 / Q5_1 blocks with 2- and 4-byte aligned
    code bytes) on the tensor-core path, k a multiple of 64 only."""
    from realizar_b200 import ops
    from realizar_b200.ops import gemm
    w, wd = _weight(n, k, qt, seed=m + n)
    assert gemm.gemm_eligible(w)
    x = torch.randn(m, k, device="cuda")
    y = gemm.gemm(w, x, splitk=splitk)
    assert ops.device_error() == 0
    xr = x.to(torch.bfloat16).float().cpu()
    ref = xr @ wd.to(torch.bfloat16).float().T
    assert float((y.cpu() - ref).abs().max() / ref.abs().max()) < 2e-2


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.BF16, QType.F16])
@pytest.mark.parametrize("m,n,k", [(5, 128, 256), (64, 200, 512), (130, 384, 1024), (33, 2560, 2560)])
def test_gemm_matches_fp32(cuda_device, qt, m, n, k):
    from realizar_b200 import ops
    from realizar_b200.ops import gemm
    w, wd = _weight(n, k, qt, seed=m + n)
    x = torch.randn(m, k, device="cuda")
    y = gemm.gemm(w, x, splitk=1)
    assert ops.device_error() == 0
    xr = x.to(torch.bfloat16).float().cpu()
    ref = xr @ wd.to(torch.bfloat16).float().T           # operands are rounded to bf16 before the tensor core
    rel = float((y.cpu() - ref).abs().max() / ref.abs().max())
    assert rel < 2e-2, rel
    ref32 = xr @ wd.T
    assert float((y.cpu() - ref32).abs().max() / ref32.abs().max()) < 3e-2


def test_gemm_epilogue_and_splitk(cuda_device):
    from realizar_b200 import ops
    from realizar_b200.ops import gemm
    m, n, k = 48, 256, 2048
    w, wd = _weight(n, k, QType.Q4_K, 9)
    x = torch.randn(m, k, device="cuda")
    bias, res = torch.randn(n, device="cuda"), torch.randn(m, n, device="cuda")
    xr = x.to(torch.bfloat16).float().cpu()
    base = xr @ wd.to(torch.bfloat16).float().T
    y = gemm.gemm(w, x, bias=bias, residual=res, act=ops.ACT_GELU, splitk=1)
    ref = torch.nn.functional.gelu(base + bias.cpu(), approximate="tanh") + res.cpu()
    assert float((y.cpu() - ref).abs().max() / ref.abs().max()) < 2e-2
    y2 = gemm.gemm(w, x, bias=bias, residual=res, splitk=4)
    ref2 = base + bias.cpu() + res.cpu()
    assert float((y2.cpu() - ref2).abs().max() / ref2.abs().max()) < 2e-2
    assert gemm.choose_splitk(2560, 10240, 64) > 1 and gemm.choose_splitk(17920 * 2, 2560, 128) == 1
    assert ops.device_error() == 0


@pytest.mark.parametrize("m", [16, 31, 64, 200, 300])
@pytest.mark.parametrize("splitk", [1, 2, 4])
def test_gemm_strided_inplace_residual(cuda_device, m, splitk):
    """The way the batched forward pass calls it: output is a column window of a wider buffer that
    already holds the residual (split-K adds into it, one split stores residual + product); rows
    and columns outside the window must stay untouched."""
    from realizar_b200 import ops
    from realizar_b200.ops import gemm as G
    n, k = 512, 1024
    w, wd = _weight(n, k, QType.Q4_K, 3)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    buf = torch.randn(m + 3, n + 40, device="cuda")
    before = buf.clone()
    win = buf[:, 8:]
    if splitk > 1:
        G.gemm_launch(G.build_gemm_params(w, x, win, m, splitk=splitk, ldy=buf.stride(0)))
    else:
        G.gemm_launch(G.build_gemm_params(w, x, win, m, residual=win, ldy=buf.stride(0), ld_res=buf.stride(0)))
    torch.cuda.synchronize()
    assert ops.lib().rlz_gemm_error(0) == 0
    ref = before[:m, 8:8 + n].cpu() + x.float().cpu() @ wd.to(torch.bfloat16).float().T
    got = buf[:m, 8:8 + n].cpu()
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-2
    assert torch.equal(buf[m:], before[m:]) and torch.equal(buf[:, :8], before[:, :8]) and torch.equal(buf[:, 8 + n:], before[:, 8 + n:])


def test_gemm_all_reduce_push_and_reduce_two_emulated_ranks(cuda_device):
    """Row-parallel GEMM with the all-reduce in the epilogue, two ranks emulated on one GPU one after
    the other (both pushes complete before the reduce runs, so nothing waits on a peer).  Each rank
    writes through 4 K splits, one of which has no K range at k = 192 and must push zeros."""
    from realizar_b200 import ops
    from realizar_b200.ops import gemm as G
    for k in (512, 192):
        m, n, world, rows_cap, splits, site, nsites = 40, 384, 2, 64, 4, 1, 3
        qt = QType.Q4_K if k % 256 == 0 else QType.BF16
        ws = [_weight(n, k, qt, 20 + r) for r in range(world)]
        xs = [torch.randn(m, k, device="cuda").to(torch.bfloat16) for _ in range(world)]
        inbox = [torch.zeros(2 * world * splits * rows_cap * n, 2, dtype=torch.int32, device="cuda") for _ in range(world)]   # 8-byte pairs
        epoch = torch.tensor([5], dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        bias = torch.randn(n, device="cuda")
        dummy = torch.zeros(m, n, device="cuda")
        for r in range(world):
            p = G.build_gemm_params(ws[r][0], xs[r], dummy, m, bias=bias if r == 0 else None)
            for q in range(world):
                p.ar_inbox[q] = inbox[q].data_ptr()
            p.ar_epoch, p.ar_row_pairs, p.ar_rank, p.ar_world, p.ar_rows, p.ar_enabled = epoch.data_ptr(), n, r, world, rows_cap, 1
            p.ar_site, p.ar_nsites, p.ar_splits = site, nsites, splits
            G.gemm_launch(p)
        torch.cuda.synchronize()
        assert ops.lib().rlz_gemm_error(0) == 0
        assert float(dummy.abs().max()) == 0.0                 # nothing is stored locally in this mode
        ref = bias.cpu() + sum(xs[r].float().cpu() @ ws[r][1].to(torch.bfloat16).float().T for r in range(world))
        for r in range(world):
            x = torch.randn(m + 2, n + 8, device="cuda")
            before = x.clone()
            ops.check(ops.lib().rlz_ll_reduce(inbox[r].data_ptr(), epoch.data_ptr(), status.data_ptr(), 1000, world * splits, rows_cap, n, site, nsites,
                                              m, n, x.data_ptr(), x.stride(0), ops.stream_ptr()), "ll_reduce")
            torch.cuda.synchronize()
            got = (x[:m, :n] - before[:m, :n]).cpu()
            assert float((got - ref).abs().max() / ref.abs().max()) < 2e-2
            assert torch.equal(x[m:], before[m:]) and torch.equal(x[:, n:], before[:, n:])
        assert int(status.item()) == 0
    # a wait that cannot complete (nobody wrote this epoch) gives up after the poll limit and reports 2003
    epoch.fill_(9)
    x = torch.zeros(m, n, device="cuda")
    ops.check(ops.lib().rlz_ll_reduce(inbox[0].data_ptr(), epoch.data_ptr(), status.data_ptr(), 50, world * splits, rows_cap, n, site, nsites, 2, 16,
                                      x.data_ptr(), x.stride(0), ops.stream_ptr()), "ll_reduce")
    torch.cuda.synchronize()
    assert int(status.item()) == 2003
    assert float(torch.ones(4, device="cuda").sum()) == 4.0     # the context is still usable


@pytest.mark.parametrize("m,k,splitk,world", [(40, 512, 1, 2), (70, 512, 2, 2), (300, 768, 1, 2), (70, 512, 2, 4), (5, 512, 1, 8), (300, 512, 1, 8)])
def test_gemm_two_shot_all_reduce_two_emulated_ranks(cuda_device, m, k, splitk, world):
    """Two-shot all-reduce of a row-parallel GEMM with two ranks emulated on one GPU, one after the other: both GEMMs store
    their tiles into the inboxes of the row owners (ownership, tile flags), then each owner's reduce kernel sums them onto
    its residual rows, applies the following norm and writes the bf16 rows into both ranks' operand buffers.  The final wait
    for the peers' rows is off (a kernel must not wait for a later launch of the same GPU); a last call with a tag nobody
    wrote shows that the bounded waits give up and report."""
    import ctypes
    from realizar_b200 import ops
    from realizar_b200.ops import gemm as G
    from realizar_b200.ops import _signatures as S
    n, splits, site, nsites = 384, 2, 1, 4
    own_rows = -(-m // world)
    own_cap, ntiles, mtiles = own_rows + 3, -(-n // 128), -(-m // 32) + 1
    ws = [_weight(n, k, QType.Q4_K if k % 256 == 0 else QType.BF16, 40 + r) for r in range(world)]
    xs = [torch.randn(m, k, device="cuda").to(torch.bfloat16) for _ in range(world)]
    local = [torch.randn(m, n, device="cuda") * 0.1 for _ in range(world)]          # each rank's local partial, added before the push
    inbox = [torch.zeros(2 * world * splits * own_cap * n, device="cuda") for _ in range(world)]
    flags = [torch.zeros(2 * world * splits * ntiles * mtiles, dtype=torch.int32, device="cuda") for _ in range(world)]
    ag = [torch.zeros(world * own_cap, dtype=torch.int32, device="cuda") for _ in range(world)]
    x0 = torch.randn(m, n, device="cuda")
    xres = [x0.clone() for _ in range(world)]
    xb = [torch.zeros(m, n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    epoch = torch.tensor([7], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bias = torch.randn(n, device="cuda")
    gamma, beta = torch.rand(n, device="cuda") + 0.5, torch.randn(n, device="cuda") * 0.1
    dummy = torch.zeros(m, n, device="cuda")
    plans = []
    for r in range(world):
        p = G.build_gemm_params(ws[r][0], xs[r], dummy, m, bias=bias if r == 0 else None, residual=local[r], splitk=splitk)
        for q in range(world):
            p.ar_inbox[q], p.rs_flags[q] = inbox[q].data_ptr(), flags[q].data_ptr()
        p.ar_epoch, p.ar_row_pairs, p.ar_rank, p.ar_world, p.ar_rows, p.ar_enabled = epoch.data_ptr(), n, r, world, own_cap, 2
        p.ar_site, p.ar_nsites, p.ar_splits = site, nsites, splits
        p.rs_own_rows, p.rs_ntiles, p.rs_mtiles = own_rows, ntiles, mtiles
        G.gemm_launch(p)
        plans.append(p)
    torch.cuda.synchronize()
    assert ops.lib().rlz_gemm_error(0) == 0 and float(dummy.abs().max()) == 0.0

    def reduce(r, push_x, to_xb, wait, limit=1000):
        nt, rows, sk = G.gemm_plan(plans[r])
        c = S.RsReduce()
        c.inbox, c.flags = inbox[r].data_ptr(), flags[r].data_ptr()
        for q in range(world):
            c.ag_flags[q], c.xpeer[q] = ag[q].data_ptr(), xres[q].data_ptr()
            c.xb[q] = xb[q].data_ptr() if to_xb else None
        c.x, c.nw, c.nb, c.epoch, c.status, c.spin_limit = xres[r].data_ptr(), gamma.data_ptr(), beta.data_ptr(), epoch.data_ptr(), status.data_ptr(), limit
        c.ldx = c.ldxb = c.ld_in = n
        c.rank, c.world, c.splits_stride, c.splits_used, c.rows_cap, c.own_rows, c.own_cap = r, world, splits, sk, own_cap, own_rows, own_cap
        c.tokens, c.n, c.nt, c.n_tiles, c.ntiles_cap, c.mtiles_cap = m, n, nt, -(-n // rows), ntiles, mtiles
        c.site, c.nsites, c.norm, c.push_x, c.wait_ag, c.eps = site, nsites, ops.NORM_LAYER, int(push_x), int(wait), 1e-5
        ops.check(ops.lib().rlz_rs_reduce(ctypes.byref(c), ops.stream_ptr()), "rs_reduce")
        torch.cuda.synchronize()

    for r in range(world):
        reduce(r, push_x=True, to_xb=True, wait=False)
    assert int(status.item()) == 0
    ref = x0.cpu() + bias.cpu() + sum(local[r].cpu() + xs[r].float().cpu() @ ws[r][1].to(torch.bfloat16).float().T for r in range(world))
    refb = torch.nn.functional.layer_norm(ref, (n,), gamma.cpu(), beta.cpu(), 1e-5)
    for q in range(world):                                    # fp32 rows and bf16 rows of BOTH owners arrived on every rank
        assert float((xres[q].cpu() - ref).abs().max() / ref.abs().max()) < 2e-2
        assert float((xb[q].float().cpu() - refb).abs().max() / refb.abs().max()) < 3e-2
    assert all(torch.equal(xres[0], xres[q]) and torch.equal(xb[0], xb[q]) for q in range(1, world))
    for q in range(world):                                    # every owned row published its tag to every rank
        got = ag[q].reshape(world, own_cap)
        for o in range(world):
            cnt = max(0, min(own_rows, m - o * own_rows))
            assert bool((got[o, :cnt] == 7 * 256 + site).all()) and bool((got[o, cnt:] == 0).all())
    # now that both owners have published, the wait for the peers' rows passes
    xres[0].copy_(x0)
    reduce(0, push_x=False, to_xb=False, wait=True)
    assert int(status.item()) == 0
    # waits that cannot complete: a new epoch that no GEMM has written (tile flags: 2004), then rows nobody gathers (2005 overrides)
    epoch.fill_(9)
    reduce(0, push_x=False, to_xb=False, wait=False, limit=50)
    assert int(status.item()) == 2004
    status.zero_()
    epoch.fill_(7)
    for q in range(world):
        ag[q].zero_()
    reduce(1, push_x=False, to_xb=False, wait=True, limit=50)          # rank 1 publishes its own rows, the other ranks' never arrive
    assert int(status.item()) == 2005
    assert float(torch.ones(4, device="cuda").sum()) == 4.0     # the context is still usable


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q6_K, QType.Q5_K, QType.BF16])
def test_gemm_wide_row_tiles(cuda_device, qt):
    """256-row CTAs (two TMEM accumulators) give the same result as 128-row CTAs, including ragged edges."""
    from realizar_b200 import ops
    from realizar_b200.ops import gemm as G
    m, n, k = 300, 600, 768
    w, wd = _weight(n, k, qt, 31)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    ref = x.float().cpu() @ wd.to(torch.bfloat16).float().T
    outs = []
    for wide in (1, 2):
        y = torch.full((m, n), float("nan"), device="cuda")
        G.gemm_launch(G.build_gemm_params(w, x, y, m, wide=wide))
        torch.cuda.synchronize()
        assert ops.lib().rlz_gemm_error(0) == 0
        assert float((y.cpu() - ref).abs().max() / ref.abs().max()) < 2e-2
        outs.append(y)
    assert float((outs[0] - outs[1]).abs().max()) < 1e-3 * float(ref.abs().max())
