"""Tensor-parallel self-test, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 -m realizar_b200.parallel.selftest --model tiny-llama

Every rank builds the same synthetic model, runs greedy decoding with the NCCL baseline and with
the in-kernel (peer-memory) collectives, and rank 0 compares both against the single-process
fp32 oracle.  Exit code 0 = all checks passed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--tokens", type=int, default=10)
    ap.add_argument("--modes", default="nccl,fused")
    ap.add_argument("--graphs", type=int, default=1)
    a = ap.parse_args(argv)
    from ..models.config import ModelConfig, ROPE_NEOX, arch_constraints, named_config
    from ..models.reference import ReferenceDecoder
    from ..models.weights import synthetic_weights
    from ..runtime.engine import DecodeEngine, EngineConfig, SamplingParams
    from .tp import make_tp_comm

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if a.model == "small-phi2":
        cfg = ModelConfig("phi2", 1280, 2, 16, 16, 80, 2560, 512, 512, 1e4, 32, ROPE_NEOX, 1e-5, None, 2,
                          arch_constraints("phi2"), parallel_residual=True, fused_qkv=True)
    elif a.model == "kq-llama":                              # every projection a K-quant: the tensor-core batched path under TP
        cfg = ModelConfig("llama", 512, 2, 8, 2, 64, 1024, 512, 512, 1e4, 64, 0, 1e-5, 1, 2, arch_constraints("llama"))
    else:
        cfg = named_config(a.model)
    w = synthetic_weights(cfg, seed=5, std=0.05)            # CPU generator: identical on every rank
    prompt = [3, 9, 27, 81, 243, 11, 5, 100, 7, 7, 19]
    ref = ReferenceDecoder(w)
    want_logits = ref.forward(prompt)[-1].numpy()
    results, ok = {}, True
    for mode in a.modes.split(","):
        comm = make_tp_comm(rank, world, dev, mode=mode)
        eng = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=256, cuda_graphs=bool(a.graphs), greedy_only=True), device=dev,
                           comm=comm, tp_rank=rank, tp_size=world)
        dist.barrier()
        toks = eng.generate(prompt, SamplingParams(max_tokens=a.tokens))
        eng.open_slot(0, 64)
        first = eng.prefill(0, prompt)
        local_logits = eng.buf.logits[0, : eng.model.vocab_local].clone()
        gathered = comm.gather_logits(local_logits[None], cfg.vocab_size)[0].cpu().numpy()
        eng.close_slot(0)
        cos = float(gathered @ want_logits / (np.linalg.norm(gathered) * np.linalg.norm(want_logits)))
        status = comm.check_status() if hasattr(comm, "check_status") else 0
        results[mode] = {"tokens": toks, "cos": cos, "first": first, "status": status, "batched_prefill": bool(eng.gemm_ok),
                         "ll_tokens": int(eng.batched().ll_tokens) if eng.gemm_ok else 0}
        ok &= cos > 0.99 and first == toks[0] and status == 0
        if eng.gemm_ok:
            # a longer prompt (beyond the one-shot limit when chunked at 128+) and a multi-token verification pass
            long_prompt = [(7 * i + 3) % cfg.vocab_size for i in range(150)]
            eng.open_slot(0, 200)
            eng.prefill(0, long_prompt)
            ll = comm.gather_logits(eng.buf.logits[0:1, : eng.model.vocab_local].clone(), cfg.vocab_size)[0].cpu().numpy()
            eng.close_slot(0)
            wl = ref.forward(long_prompt)[-1].numpy()
            cos2 = float(ll @ wl / (np.linalg.norm(ll) * np.linalg.norm(wl)))
            results[mode]["cos_long"] = cos2
            ok &= cos2 > 0.99 and (comm.check_status() if hasattr(comm, "check_status") else 0) == 0
            # multi-token verification with more rows than max_batch: several head passes (and candidate exchanges) in one call
            eng.open_slot(0, 64)
            eng.prefill(0, prompt)
            ver = eng.forward_tokens(0, [5, 9, 13, 2, 8])
            eng.close_slot(0)
            v = torch.tensor(ver, device=dev)
            v0 = v.clone()
            dist.broadcast(v0, 0)
            results[mode]["verify"] = ver
            ok &= bool((v == v0).all()) and (comm.check_status() if hasattr(comm, "check_status") else 0) == 0
        t = torch.tensor(toks, device=dev)
        t0 = t.clone()
        dist.broadcast(t0, 0)
        ok &= bool((t == t0).all())                          # every rank generated the same tokens
        # non-greedy sampling: candidates of the vocabulary slices exchanged over peer memory (fused) against the gathered row
        eng.close()
        del eng
        torch.cuda.synchronize()
        dist.barrier()
        sampled = {}
        for sharded in (("1", "0") if mode == "fused" else ("0",)):
            os.environ["RLZ_SHARDED_SAMPLING"] = sharded
            eng2 = DecodeEngine(w, EngineConfig(max_batch=2, max_seq_len=256, cuda_graphs=bool(a.graphs), greedy_only=False, seed=11), device=dev,
                                comm=comm, tp_rank=rank, tp_size=world)
            sampled[sharded] = eng2.generate(prompt, SamplingParams(max_tokens=a.tokens, temperature=0.8, top_k=50, top_p=0.9))
            st = torch.tensor(sampled[sharded], device=dev)
            st0 = st.clone()
            dist.broadcast(st0, 0)
            ok &= bool((st == st0).all()) and (comm.check_status() if hasattr(comm, "check_status") else 0) == 0
            eng2.close()
            del eng2
        os.environ.pop("RLZ_SHARDED_SAMPLING", None)
        results[mode]["sampled"] = sampled
        if len(sampled) == 2:
            ok &= sampled["1"] == sampled["0"]
        comm.close()
        torch.cuda.synchronize()
    modes = list(results)
    if len(modes) == 2:
        ok &= results[modes[0]]["tokens"] == results[modes[1]]["tokens"]
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"ok": bool(flag.item()), "world": world, "model": a.model, "results": results,
                          "oracle_argmax": int(want_logits.argmax())}))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if flag.item() else 1


if __name__ == "__main__":
    sys.exit(main())
