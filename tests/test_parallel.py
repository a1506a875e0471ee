"""Parallel configuration, mock communicator arithmetic, weight sharding for tensor parallelism
and a two-process gloo run of the torch communicator."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from realizar_b200 import quant
from realizar_b200.models.decoder import shard_cols, shard_rows
from realizar_b200.models.weights import QTensor
from realizar_b200.parallel.config import (DistributedContext, MockCommunicator, ParallelConfig, ParallelError, PipelineParallel,
                                           ReduceOp, TensorParallel, ZeroOffload)
from realizar_b200.quant import QType


def test_rank_decomposition_tp_fastest():
    c = ParallelConfig(tp_size=4, pp_size=2, dp_size=2, rank=13)
    assert (c.world_size, c.tp_rank, c.pp_rank, c.dp_rank) == (16, 1, 1, 1)
    assert c.tp_group() == [12, 13, 14, 15]
    with pytest.raises(ParallelError):
        ParallelConfig(2, 1, 1, rank=2)
    assert not ParallelConfig().is_distributed


def test_mock_collectives():
    m = MockCommunicator(4, 1)
    t = torch.arange(8.0).reshape(4, 2)
    assert torch.equal(m.all_reduce(t), t * 4) and torch.equal(m.all_reduce(t, ReduceOp.MAX), t)
    assert m.all_gather(t).shape == (16, 2)
    assert torch.equal(m.reduce_scatter(t), t[1:2] * 4)
    m.barrier()
    assert m.calls[-1] == "barrier"


def test_tensor_parallel_linear_matches_dense():
    torch.manual_seed(0)
    W1, W2, b2, x = torch.randn(16, 8), torch.randn(8, 16), torch.randn(8), torch.randn(3, 8)
    want = (x @ W1.T) @ W2.T + b2
    parts = []
    for r in range(4):
        tp = TensorParallel(4, r, MockCommunicator(1, 0))       # identity all-reduce: we sum by hand
        h = tp.column_parallel_linear(x, tp.shard_columns(W1))
        parts.append(tp.row_parallel_linear(h, tp.shard_rows(W2), b2))
    assert torch.allclose(sum(parts), want, atol=1e-5)            # bias only from rank 0


def test_pipeline_partition_and_bubble():
    p = PipelineParallel(4, 1, 30, num_micro_batches=8)
    assert [p.layer_range(s) for s in range(4)] == [(0, 8), (8, 16), (16, 23), (23, 30)]
    assert abs(p.bubble_ratio - 3 / 11) < 1e-9 and p.micro_batch_size(20) == 3
    assert p.stats().layers_per_stage == [8, 8, 7, 7]
    ctx = DistributedContext.create(tp=2, pp=2, rank=3, num_layers=8)
    assert ctx.is_distributed and ctx.tp.rank == 1 and ctx.pp.stage == 1
    assert ZeroOffload(True, True, param_fraction_on_gpu=0.5).memory_savings_ratio() == pytest.approx(0.55)


@pytest.mark.parametrize("qt,k,tp", [(QType.Q4_K, 2560, 8), (QType.Q5_K, 1280, 4), (QType.Q6_K, 2560, 8), (QType.Q8_0, 640, 4), (QType.Q4_K, 1024, 2)])
def test_row_parallel_shards_sum_to_full_product(qt, k, tp):
    """Column shards keep whole blocks and silence foreign sub-blocks; partial products add up."""
    n = 12
    w = (np.random.default_rng(1).standard_normal((n, k)) * 0.02).astype(np.float32)
    t = QTensor(int(qt), (n, k), quant.quantize(w, qt))
    full = t.to_f32()
    x = np.random.default_rng(2).standard_normal(k).astype(np.float32)
    total = np.zeros(n, np.float32)
    step = k // tp
    for r in range(tp):
        sh, cover0 = shard_cols(t, r * step, (r + 1) * step)
        xs = np.zeros(sh.shape[1], np.float32)
        xs[r * step - cover0: (r + 1) * step - cover0] = x[r * step:(r + 1) * step]
        junk = np.where(xs == 0, 123.0, xs).astype(np.float32)          # garbage outside the owned range must not matter
        assert np.allclose(sh.to_f32() @ xs, sh.to_f32() @ junk, atol=1e-4)
        total += sh.to_f32() @ xs
    assert np.allclose(total, full @ x, atol=1e-4)
    rows = shard_rows(t, 4, 8)
    assert np.array_equal(rows.to_f32(), full[4:8])


def test_torch_communicator_two_gloo_ranks(tmp_path):
    script = tmp_path / "w.py"
    script.write_text("""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from realizar_b200.parallel.config import TorchCommunicator, TensorParallel, ReduceOp
dist.init_process_group('gloo')
c = TorchCommunicator()
r = c.rank
t = torch.full((4, 2), float(r + 1))
assert torch.equal(c.all_reduce(t), torch.full((4, 2), 3.0))
assert torch.equal(c.all_reduce(t, ReduceOp.MAX), torch.full((4, 2), 2.0))
assert c.all_gather(t).shape == (8, 2)
assert torch.equal(c.reduce_scatter(t), torch.full((2, 2), 3.0))
torch.manual_seed(0)
W, x = torch.randn(6, 8), torch.randn(2, 8)
tp = TensorParallel(2, r, c)
y = tp.row_parallel_linear(x[:, r * 4:(r + 1) * 4], tp.shard_rows(W))
assert torch.allclose(y, x @ W.T, atol=1e-5)
c.barrier()
dist.destroy_process_group()
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]


def test_tensor_parallel_serving_proxy_two_gloo_ranks(tmp_path):
    """Rank 0 runs the serving loop over a leader proxy, rank 1 follows: both (toy) engines must see the same calls with
    the same arguments - slots, sampling parameters with penalties and logit_bias, prompt chunks, decode steps, token masks,
    scoring passes - and rank 1 leaves its loop when the leader shuts down."""
    script = tmp_path / "tp.py"
    script.write_text("""
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from realizar_b200.parallel.tp_serving import TpLeaderEngine, follower_loop
from realizar_b200.runtime.scheduler import FakeEngine, Request, ServingEngine
dist.init_process_group('gloo')
rank = dist.get_rank()
group = dist.new_group(backend='gloo')
eng = FakeEngine(max_batch=2, vocab=50, fail_after=7)      # the 8th decode step fails on EVERY rank (same call sequence everywhere)
if rank == 0:
    lead = TpLeaderEngine(eng, group)
    sv = ServingEngine(lead).start()
    class Mask:
        def __init__(self): self.n = 0
        def mask(self): return [i in (7, 9) for i in range(50)]
        def accept_token(self, t): self.n += 1; return True
    r1 = sv.generate([1, 2, 3], max_tokens=4, temperature=0.7, top_k=5, presence_penalty=0.5, logit_bias={4: -3.0}, timeout=30)
    r2 = sv.generate([10, 11], max_tokens=3, token_masker=Mask(), timeout=30)
    sc = sv.call_on_engine(lambda e: e.score_tokens([5, 6, 7], want_embedding=True))
    assert r1.output == [4, 5, 6, 7] and r2.output == [7, 7, 7] and len(sc['logprobs']) == 2, (r1.output, r2.output, sc)
    # a step that fails on every rank (same call sequence, same counter): the loop latches, the followers stop executing,
    # the reset command brings all ranks back in step and serving goes on
    import time
    assert eng.steps == 5
    bad = sv.generate([1, 2, 3], max_tokens=8, timeout=30)
    assert bad.error is not None
    for _ in range(200):
        if sv.health != 'ok' and not sv._thread.is_alive():
            break
        time.sleep(0.01)
    assert sv.health == 'unhealthy'
    assert sv.recover() and sv.health == 'ok'
    r3 = sv.generate([20, 21], max_tokens=3, timeout=30)
    assert r3.output == [22, 23, 24], r3.output
    sv.stop()
    lead.shutdown(leave=False)
else:
    n = follower_loop(eng, group)
    assert n > 0
calls = [c for c in eng.calls]
gathered = [None, None]
dist.all_gather_object(gathered, json.dumps(calls))
assert gathered[0] == gathered[1], (gathered[0][:400], gathered[1][:400])
sp = getattr(eng, 'sampling_log', [])
assert any(v.presence_penalty == 0.5 and v.logit_bias == {4: -3.0} and v.top_k == 5 and abs(v.temperature - 0.7) < 1e-9 for v in sp), sp
dist.barrier()
dist.destroy_process_group()
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29549", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]


def test_rank_failure_is_detected_by_the_survivor(tmp_path):
    """Failure drill on CPU ranks: rank 1 leaves between steps (no collective in flight); rank 0 learns of it
    through a heartbeat in the rendezvous store before its next collective, and a collective that is attempted
    anyway ends with a time-out error instead of hanging."""
    script = tmp_path / "f.py"
    script.write_text("""
import datetime, os, sys, time, torch, torch.distributed as dist
sys.path.insert(0, %r)
rank = int(os.environ['RANK'])
store = dist.TCPStore('127.0.0.1', 29547, 2, rank == 0, timeout=datetime.timedelta(seconds=20))
dist.init_process_group('gloo', store=store, rank=rank, world_size=2, timeout=datetime.timedelta(seconds=3))
t = torch.ones(4) * (rank + 1)
dist.all_reduce(t)                      # step 1: both ranks healthy
assert t[0] == 3
store.set(f'hb{rank}', str(time.time()))
if rank == 1:
    store.set('left1', '1')             # announce, then leave between steps
    os._exit(0)
store.wait(['left1'])
# host-side detection before the next launch: the peer announced that it left (a stale heartbeat works the same way)
peer_alive = False
detected_by_timeout = False
try:                                    # and a collective issued regardless gives up after the group time-out
    dist.all_reduce(torch.ones(4))
except Exception as e:
    detected_by_timeout = True
print('RESULT', peer_alive, detected_by_timeout, flush=True)
os._exit(0 if (not peer_alive and detected_by_timeout) else 3)
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29546", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert procs[1].returncode == 0
    assert procs[0].returncode == 0, outs[0][0][-1000:] + outs[0][1][-2000:]
    assert "RESULT False True" in outs[0][0]
