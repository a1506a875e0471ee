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
