#!/usr/bin/env python
"""Headline benchmark: batch-1 decode tokens/s of a Phi-2-shaped decoder (32 layers, hidden 2560,
32 heads x 80, partial rotary 32, LayerNorm, parallel attention+MLP, GELU, vocab 51200) with
random-init weights quantised to the Q4_K_M mixture, after a 512-token prompt, on N GPUs
(tensor parallel) of one node.

    python bench.py --gpus 1 --steps 256 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 4 --steps 256 --warmup 8

A step is one decode token for the whole batch.  `value` is measured with CUDA events around
K graph replays with device-side token feedback; `e2e` is the same loop through the public
streaming API (pinned-host token in, sampled token out, every step).
Rank 0 prints one JSON line.
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
    print(json.dumps({"impl": "reference", "unavailable": "reference is a Rust crate: pip install fails (neither setup.py nor "
                      "pyproject.toml), no cargo/rustc and its trueno* crates are not vendored", "n_gpus": args.gpus}))
    return 0


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
    max_seq = ((args.prompt_len + 2 * (K + W) + 64 + 15) // 16) * 16
    t0 = time.time()
    weights = synthetic_weights(cfg, scheme=args.scheme, seed=0, device=dev)      # same seed on every rank
    eng = DecodeEngine(weights, EngineConfig(max_batch=B, max_seq_len=max_seq, cuda_graphs=not args.no_graphs, pdl=not args.no_pdl,
                                             greedy_only=True), device=dev, comm=comm, tp_rank=rank, tp_size=world)
    total_weight_bytes = weights.total_bytes()
    del weights
    torch.cuda.empty_cache()
    load_s = time.time() - t0

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # ---- prompt: uniform random ids, prefilled through the engine ---------------------------
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (B, args.prompt_len), generator=g)
    for b in range(B):
        eng.open_slot(b, max_seq)
    # warm the prefill path once with a full-length scratch prompt in slot 0 (kernel attributes, allocator, and the
    # first NCCL collective of that message size under tensor parallelism), then time TTFT
    eng.prefill(0, [int(t) for t in torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g)])
    eng.close_slot(0)
    eng.open_slot(0, max_seq)
    sync_all()
    profile_prefill = os.environ.get("RLZ_PROFILE_REGION") == "prefill"   # `ncu --profile-from-start off`: capture the timed prefill only
    if profile_prefill:
        torch.cuda.cudart().cudaProfilerStart()
    t0 = time.time()
    first = [eng.prefill(b, [int(t) for t in prompts[b]]) for b in range(B)]
    torch.cuda.synchronize(dev)
    prefill_s = time.time() - t0
    if profile_prefill:
        torch.cuda.cudart().cudaProfilerStop()

    # ---- device-timed decode: graph replays with device-side feedback ---------------------------
    pos0 = eng.slots[0].position
    eng.buf.tokens[:B].copy_(torch.tensor(first, dtype=torch.int32))
    eng.buf.positions[:B].fill_(pos0)
    for b in range(B):
        eng._ensure_pages(b, max_seq)
    for _ in range(W):
        eng.run_step(B)
        eng.advance(B)
    sync_all()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    profile_region = os.environ.get("RLZ_PROFILE_REGION") in ("1", "decode")     # `ncu --profile-from-start off`: capture the timed steps only
    if profile_region:
        torch.cuda.cudart().cudaProfilerStart()
    e0.record()
    for _ in range(K):
        eng.run_step(B)
        eng.advance(B)
    e1.record()
    sync_all()
    if profile_region:
        torch.cuda.cudart().cudaProfilerStop()
    clocks = sampler.stop()
    eager_launches = ops.launch_count() - l0
    ms = e0.elapsed_time(e1)
    for b in range(B):
        eng.slots[b].position = pos0 + W + K
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    tok_s = B * K / (ms / 1e3)
    launches = (eng.kernels_per_step(eng.bucket_for(B)) + 1) * K

    # ---- end-to-end: public streaming path, pinned token in / sampled token out every step -----
    cur = {b: int(eng.buf.sampled[b]) for b in range(B)}
    for _ in range(3):
        out = eng.feed(cur)
        cur = {b: int(out[b]) for b in range(B)}
    sync_all()
    t0 = time.perf_counter()
    for _ in range(K):
        out = eng.feed(cur)
        cur = {b: int(out[b]) for b in range(B)}
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t)
    e2e_tok_s = B * K / e2e_s

    if rank == 0:
        pub = PUBLISHED.get(args.model)
        line = {
            "metric": "decode tok/s (bs=%d, %s)" % (B, args.scheme), "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(tok_s / pub, 3) if pub else None, "dtype": "q4_k_m weights, int8/fp32 activations, bf16 KV",
            "data": "synthetic (random-init N(0,0.02) weights, uniform-random prompt ids)",
            "config": {"model": args.model + "-shaped", "global_batch": B, "seq_len": args.prompt_len + W + K, "prompt_len": args.prompt_len,
                       "parallelism": "tp%d" % world, "tp_comm": args.tp_comm if world > 1 else None,
                       "l2": "weights per GPU (%.0f MB) exceed L2; no flush" % (eng.model.weight_bytes() / 1e6),
                       "cuda_graphs": not args.no_graphs, "pdl": eng.pdl, "kernels_per_step": eng.kernels_per_step(eng.bucket_for(B)) + 1,
                       "baseline": "published %s tok/s on RTX 4090 (reference README)" % pub},
            "clocks": clocks,
            "e2e": {"value": round(e2e_tok_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": int(launches),
            "aux": {"load_s": round(load_s, 2), "ttft_ms_prompt%d" % args.prompt_len: round(prefill_s * 1e3 / B, 2), "prefill_path": "tcgen05 gemm" if eng.gemm_ok else "serial decode kernels", "weight_bytes_total": int(total_weight_bytes),
                    "launch_calls_outside_graphs": int(eager_launches)},
        }
        print(json.dumps(line))
    if world > 1:
        # leave without tearing NCCL down: communicator destruction after graph-captured collectives can block
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
