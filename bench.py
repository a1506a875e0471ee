#!/usr/bin/env python
"""Headline benchmark: batch-1 decode tokens/s of a Phi-2-shaped decoder (32 layers, hidden 2560,
32 heads x 80, partial rotary 32, LayerNorm, parallel attention+MLP, GELU, vocab 51200) with
random-init weights quantised to the Q4_K_M mixture, after a 512-token prompt, on N GPUs
(tensor parallel) of one node.

    python bench.py --gpus 1 --steps 256 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 4 --steps 256 --warmup 8

A step is one decode token for the whole batch.  `value` is the median over `--repeats` regions
of exactly K graph replays with device-side token feedback, each timed with CUDA events (max over
ranks); `e2e` is the same loop through the public streaming API (pinned-host token in, sampled
token out, every step).  The same line carries `aux.bs64` (the batch-64 half of the metric on the
same engine), `aux.ttft_ms_p50` over at least five distinct prompts and, under tensor
parallelism, `aux.nccl_arm` (the same steps with NCCL all-reduces) and `aux.tp_parity` (cosine
of the first decode step's logits between the two communicators).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

PUBLISHED = {"phi-2": 276.0, "llama-3-8b": 110.7, "llama-3-70b": None, "qwen2.5-0.5b": None}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="phi-2")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--scheme", default="Q4_K_M")
    ap.add_argument("--tp-comm", default="fused", choices=["fused", "nccl"], help="row-parallel all-reduce: in-kernel peer stores or NCCL")
    ap.add_argument("--repeats", type=int, default=10, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--aux-batch", type=int, default=64, help="also report device-timed decode at this batch (aux.bsN); 0 = off")
    ap.add_argument("--no-nccl-arm", action="store_true", help="tensor parallel: skip the NCCL all-reduce arm and the parity figure")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
                 "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80)}
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = get(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.ok:
            self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def reference_arm(args):
    # The reference is a Rust crate (no setup.py / pyproject.toml, no cargo toolchain or vendored crates
    # in this image), so installing it with pip fails and there is nothing to run.
    if int(os.environ.get("RANK", "0")) == 0:               # one line per job, also when every rank of a multi-GPU launch gets here
        print(json.dumps({"impl": "reference", "unavailable": "reference is a Rust crate: pip install fails (neither setup.py nor "
                          "pyproject.toml), no cargo/rustc and its trueno* crates are not vendored", "n_gpus": args.gpus}))
    return 0


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2] if len(s) % 2 else 0.5 * (s[len(s) // 2 - 1] + s[len(s) // 2])


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from realizar_b200 import ops
    from realizar_b200.models.config import named_config
    from realizar_b200.models.weights import synthetic_weights
    from realizar_b200.runtime.engine import DecodeEngine, EngineConfig, SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run (WORLD_SIZE={world})", file=sys.stderr)
            return 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from realizar_b200.parallel.tp import make_tp_comm
        comm = make_tp_comm(rank, world, dev, mode=args.tp_comm)

    cfg = named_config(args.model)
    K, W, B = args.steps, max(3, args.warmup), args.batch
    R = max(1, args.repeats)
    BIG = max(B, args.aux_batch) if args.aux_batch > 0 else B       # one engine serves the headline batch and the bs=64 figure
    max_seq = ((args.prompt_len + (K + W) + 64 + 15) // 16) * 16
    t0 = time.time()
    weights = synthetic_weights(cfg, scheme=args.scheme, seed=0, device=dev)      # same seed on every rank
    ecfg = EngineConfig(max_batch=BIG, max_seq_len=max_seq, cuda_graphs=not args.no_graphs, pdl=not args.no_pdl, greedy_only=True)
    eng = DecodeEngine(weights, ecfg, device=dev, comm=comm, tp_rank=rank, tp_size=world)
    total_weight_bytes = weights.total_bytes()
    load_s = time.time() - t0

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- prompts: uniform random ids, prefilled through the engine; TTFT = wall time of one prefill call ----------
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (BIG, args.prompt_len), generator=g)

    def prefill_all(e, n):
        """Open slots 0..n-1 and run their prompts; returns (first tokens, per-prompt wall times in ms)."""
        firsts, times = [], []
        for b in range(n):
            e.open_slot(b, max_seq)
            torch.cuda.synchronize(dev)
            t = time.perf_counter()
            firsts.append(e.prefill(b, [int(x) for x in prompts[b]]))
            torch.cuda.synchronize(dev)
            times.append((time.perf_counter() - t) * 1e3)
        return firsts, times

    # warm the prefill path once with a scratch prompt (kernel attributes, allocator, first collectives of that size)
    eng.open_slot(0, max_seq)
    eng.prefill(0, [int(t) for t in torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g)])
    eng.close_slot(0)
    sync_all()
    n_ttft = max(B, min(BIG, 8))                         # at least 5 distinct prompts for the TTFT median when the engine has the slots
    first, ttft = prefill_all(eng, n_ttft)
    for b in range(B, n_ttft):
        eng.close_slot(b)
    pos0 = eng.slots[0].position

    def timed_decode(e, nb, firsts, repeats):
        """Device-timed decode of slots 0..nb-1: `repeats` regions of exactly K graph-replayed steps with device-side token
        feedback, each region restarting at the position after the prompt (+ W warm-up steps).  Returns ms per region."""
        for b in range(nb):
            e._ensure_pages(b, max_seq)
        out = []
        for _ in range(repeats):
            e.buf.tokens[:nb].copy_(torch.tensor(firsts[:nb], dtype=torch.int32))
            e.buf.positions[:nb].fill_(pos0)
            for _ in range(W):
                e.run_step(nb)
                e.advance(nb)
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                e.run_step(nb)
                e.advance(nb)
            e1.record()
            sync_all()
            out.append(max_over_ranks(e0.elapsed_time(e1)))
        return out

    # ---- headline: device-timed decode at batch B ----------------------------------------------------------------
    timed_decode(eng, B, first, 1)                       # graph capture and first replays outside the sampled region
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ops.launch_count()
    profile_region = os.environ.get("RLZ_PROFILE_REGION") in ("1", "decode")     # `ncu --profile-from-start off`: capture the timed steps only
    if profile_region:
        torch.cuda.cudart().cudaProfilerStart()
    regions = timed_decode(eng, B, first, R)
    if profile_region:
        torch.cuda.cudart().cudaProfilerStop()
    eager_launches = ops.launch_count() - l0
    ms = median(regions)
    tok_s = B * K / (ms / 1e3)
    launches = (eng.kernels_per_step(eng.bucket_for(B)) + 1) * K

    # ---- end-to-end: public streaming path, pinned token in / sampled token out every step ------------------------
    def timed_e2e(e, nb, firsts, repeats):
        out = []
        for _ in range(repeats):
            for b in range(nb):
                e.slots[b].position = pos0
            cur = {b: int(firsts[b]) for b in range(nb)}
            for _ in range(W):
                o = e.feed(cur)
                cur = {b: int(o[b]) for b in range(nb)}
            sync_all()
            t = time.perf_counter()
            for _ in range(K):
                o = e.feed(cur)
                cur = {b: int(o[b]) for b in range(nb)}
            torch.cuda.synchronize(dev)
            out.append(max_over_ranks(time.perf_counter() - t))
        return out

    e2e_regions = timed_e2e(eng, B, first, R)
    clocks = sampler.stop()
    e2e_tok_s = B * K / median(e2e_regions)

    aux = {"load_s": round(load_s, 2), "ttft_ms_p50": round(median(ttft), 2), "ttft_ms_all": [round(t, 2) for t in ttft],
           "ttft_prompts": len(ttft), "prefill_path": "tcgen05 gemm" if eng.gemm_ok else "serial decode kernels",
           "weight_bytes_total": int(total_weight_bytes), "launch_calls_outside_graphs": int(eager_launches)}

    # ---- aux: the bs = 64 half of the metric on the same engine (all slots prefilled, device-timed the same way) ------
    if BIG > B:
        for b in range(B):
            eng.close_slot(b)
        big_first, _ = prefill_all(eng, BIG)
        timed_decode(eng, BIG, big_first, 1)
        big = timed_decode(eng, BIG, big_first, max(3, R // 3))
        aux["bs%d" % BIG] = {"value": round(BIG * K / (median(big) / 1e3), 1), "unit": "tok/s", "ms_per_step": round(median(big) / K, 4),
                             "repeats": len(big), "kernels_per_step": eng.kernels_per_step(eng.bucket_for(BIG)) + 1}

    # ---- aux under tensor parallelism: the same K steps with NCCL all-reduces, and the agreement of the two paths -----
    if world > 1 and args.tp_comm == "fused" and not args.no_nccl_arm:
        from realizar_b200.parallel.tp import make_tp_comm
        ncomm = make_tp_comm(rank, world, dev, mode="nccl")
        neng = DecodeEngine(weights, EngineConfig(max_batch=B, max_seq_len=max_seq, cuda_graphs=not args.no_graphs, pdl=not args.no_pdl,
                                                  greedy_only=True), device=dev, comm=ncomm, tp_rank=rank, tp_size=world)
        nfirst, _ = prefill_all(neng, B)
        timed_decode(neng, B, nfirst, 1)
        nreg = timed_decode(neng, B, nfirst, max(3, R // 2))
        aux["nccl_arm"] = {"value": round(B * K / (median(nreg) / 1e3), 2), "unit": "tok/s", "ms_per_step": round(median(nreg) / K, 5), "repeats": len(nreg)}
        # parity: logits of the first decode step after the same prompt, fused vs NCCL communicator (this rank's vocabulary shard)
        for e in (eng, neng):
            for b in range(e.cfg.max_batch):
                e.close_slot(b)
            e.open_slot(0, max_seq)
            tok = e.prefill(0, [int(x) for x in prompts[0]])
            e.feed({0: int(tok)})
        a_, b_ = eng.buf.logits[0, : eng.model.vocab_local].double(), neng.buf.logits[0, : neng.model.vocab_local].double()
        stats = torch.stack([(a_ * b_).sum(), (a_ * a_).sum(), (b_ * b_).sum()])
        dist.all_reduce(stats)
        aux["tp_parity"] = round(float(stats[0] / (stats[1].sqrt() * stats[2].sqrt() + 1e-30)), 6)
        neng.close()
        ncomm.close()

    if rank == 0:
        pub = PUBLISHED.get(args.model)
        line = {
            "metric": "decode tok/s (bs=%d, %s)" % (B, args.scheme), "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 5), "repeats": len(regions),
            "ms_per_step_min": round(min(regions) / K, 5), "ms_per_step_max": round(max(regions) / K, 5),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(tok_s / pub, 3) if pub else None, "dtype": "q4_k_m weights, int8/fp32 activations, bf16 KV",
            "data": "synthetic (random-init N(0,0.02) weights, uniform-random prompt ids)",
            "config": {"model": args.model + "-shaped", "global_batch": B, "seq_len": args.prompt_len + W + K, "prompt_len": args.prompt_len,
                       "parallelism": "tp%d" % world, "tp_comm": args.tp_comm if world > 1 else None,
                       "l2": "weights per GPU (%.0f MB) exceed L2; no flush" % (eng.model.weight_bytes() / 1e6),
                       "timing": "median over %d regions of %d steps, each region after %d warm-up steps" % (len(regions), K, W),
                       "cuda_graphs": not args.no_graphs, "pdl": eng.pdl, "kernels_per_step": eng.kernels_per_step(eng.bucket_for(B)) + 1,
                       "baseline": "published %s tok/s on RTX 4090 (reference README)" % pub},
            "clocks": clocks,
            "e2e": {"value": round(e2e_tok_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 8 * BIG, "d2h_bytes_per_step": 4 * B,
                    "repeats": len(e2e_regions)},
            "gpu_launches": int(launches),
            "aux": aux,
        }
        print(json.dumps(line))
        sys.stdout.flush()
    # ---- orderly teardown: captured graphs hold communicator work, so they go first -------------------------------
    eng.close()
    if comm is not None:
        comm.close()
    if world > 1:
        torch.cuda.synchronize(dev)
        dist.barrier()
        guard = threading.Timer(60.0, lambda: (sys.stderr.write("bench.py: process-group teardown did not finish in 60 s; leaving\n"), os._exit(0)))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
