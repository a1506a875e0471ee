"""Tensor parallelism on the GPU: the in-kernel all-reduce on one GPU (self-loop and a bounded
wait that runs out), and 2-rank runs as child processes when two GPUs are present."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from realizar_b200 import quant
from realizar_b200.quant import QType

pytestmark = pytest.mark.gpu


def _weight(n, k, qt, seed):
    from realizar_b200 import ops
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    q = quant.quantize(w, qt)
    return ops.upload_weight(q, qt, n, k, "cuda"), torch.from_numpy(quant.dequantize(q, qt, (n, k)))


def test_fused_allreduce_single_rank_self_loop(cuda_device):
    """world = 1: the kernel pushes into its own inbox, sees its own flag and adds the residual."""
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn
    from realizar_b200.parallel.tp import FusedTpComm
    n, k, B = 640, 512, 2
    w, wd = _weight(n, k, QType.Q4_K, 3)
    comm = FusedTpComm(0, 1, "cuda", spin_limit=1_000_000)
    comm.allocate(2, n, max_batch=4)
    x = torch.randn(B, k, device="cuda")
    res = torch.randn(B, n, device="cuda")
    bias = torch.randn(n, device="cuda")
    for step in range(3):                       # both parities and a reused slot
        comm.begin_step()
        y = res.clone()
        p = ops.build_gemv_params([VecIn(x, k)], [MatOut([(w, 0)], bias=bias, residual=True)], y, B, residual=y, ar=comm.ar_desc(step % 2))
        ops.gemv_launch(p)
        torch.cuda.synchronize()
        ref = x.cpu() @ wd.T + bias.cpu() + res.cpu()
        assert float((y.cpu() - ref).abs().max() / ref.abs().max()) < 0.02
    assert comm.check_status() == 0
    # candidate exchange with one rank is the identity
    val, idx, out = torch.tensor([1.5, -2.0], device="cuda"), torch.tensor([7, 9], device="cuda", dtype=torch.int32), torch.zeros(2, device="cuda", dtype=torch.int32)
    comm.select_greedy(val, idx, out, 2)
    assert out.cpu().tolist() == [7, 9]
    comm.close()


def test_peer_wait_runs_out_and_reports_status(cuda_device):
    """A flag that nothing sets: the bounded wait expires, the kernel records 2001 and returns."""
    from realizar_b200 import ops
    from realizar_b200.ops import MatOut, VecIn, _signatures as S
    n, k = 256, 256
    w, _ = _weight(n, k, QType.Q4_K, 4)
    world = 2
    inbox = [torch.zeros(2 * world * 4 * n * 2, device="cuda", dtype=torch.int32) for _ in range(world)]   # "rank 1" memory is a second local buffer
    epoch = torch.ones(1, device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    ar = S.GemvAr()
    for r in range(world):
        ar.inbox[r] = inbox[r].data_ptr()
    ar.epoch, ar.status, ar.spin_limit = epoch.data_ptr(), status.data_ptr(), 2000
    ar.rank, ar.world, ar.enabled, ar.n = 0, world, 1, n
    x, y = torch.randn(1, k, device="cuda"), torch.zeros(1, n, device="cuda")
    ops.gemv_launch(ops.build_gemv_params([VecIn(x, k)], [MatOut([(w, 0)])], y, 1, ar=ar))
    torch.cuda.synchronize()                                # returns: nobody played rank 1, the wait ran out
    assert int(status.item()) == 2001
    par = 1                                                 # epoch 1 -> parity 1
    pairs = inbox[1].view(2, world, 4 * n, 2)               # [parity][rank][element][value bits, epoch]
    assert bool((pairs[par, 0, :n, 1] == 1).all())          # our epoch-tagged values did reach the peer's inbox
    assert torch.isfinite(y).all()
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def _run_selftest(nproc, model, extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", "-m", "realizar_b200.parallel.selftest", "--model", model, *extra]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.mark.parametrize("model", ["tiny-llama", "small-phi2", "kq-llama"])
def test_two_rank_tp_matches_oracle(cuda_device, model):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run_selftest(2, model)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert '"ok": true' in r.stdout
