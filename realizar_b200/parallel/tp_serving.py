"""Tensor-parallel serving: rank 0 owns HTTP and the scheduler, every rank runs the identical engine step.

The serving loop talks to its engine through a handful of calls (open / close a slot, set sampling, run a prompt chunk, run a
decode step, score tokens, self-speculative helpers).  ``TpLeaderEngine`` wraps rank 0's ``DecodeEngine`` and, before it executes
a call, broadcasts it to the follower ranks over a CPU (gloo) side group - a fixed header ``[op, slot, n_ints, n_floats]`` and a
payload of integers / floats only when there is one, so a decode step costs one small broadcast.  ``follower_loop`` on the other
ranks executes the same calls on their engines; the collectives inside the kernels (peer-memory all-reduces, candidate exchange)
then line up rank for rank.  Random numbers for sampling come from generators seeded alike on every rank, and every rank sees
the same sequence of calls, so sampled tokens agree without exchanging them.

The reference's serving boot and batch scheduler are single-GPU (src/cli/mod_server_commands.rs:576-660,
src/api/cuda_batch_scheduler.rs:94-460); this is their tensor-parallel counterpart.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import logging

import numpy as np
import torch
import torch.distributed as dist

log = logging.getLogger("realizar_b200.tp_serving")

OP_STOP, OP_OPEN, OP_CLOSE, OP_SAMPLING, OP_PREFILL, OP_FEED, OP_SCORE, OP_MASK, OP_DRAFT, OP_FORWARD, OP_ROLLBACK, OP_RESET = range(12)


class _Channel:
    """Command channel from rank 0 to the followers: int64 header, then int64 and float64 payloads when present."""

    def __init__(self, group, src: int = 0):
        self.group, self.src = group, src

    def send(self, op: int, slot: int = -1, ints: Sequence[int] = (), floats: Sequence[float] = ()) -> None:
        hdr = torch.tensor([op, slot, len(ints), len(floats)], dtype=torch.int64)
        dist.broadcast(hdr, self.src, group=self.group)
        if len(ints):
            dist.broadcast(torch.as_tensor(np.asarray(ints, dtype=np.int64)), self.src, group=self.group)
        if len(floats):
            dist.broadcast(torch.as_tensor(np.asarray(floats, dtype=np.float64)), self.src, group=self.group)

    def recv(self):
        hdr = torch.zeros(4, dtype=torch.int64)
        dist.broadcast(hdr, self.src, group=self.group)
        op, slot, ni, nf = (int(v) for v in hdr)
        ints = torch.zeros(ni, dtype=torch.int64)
        floats = torch.zeros(nf, dtype=torch.float64)
        if ni:
            dist.broadcast(ints, self.src, group=self.group)
        if nf:
            dist.broadcast(floats, self.src, group=self.group)
        return op, slot, [int(v) for v in ints], [float(v) for v in floats]


def _sampling_to_wire(sp):
    lb = sp.logit_bias or {}
    ints = [int(sp.top_k), int(sp.max_tokens), len(lb)] + [int(k) for k in lb]
    floats = [float(sp.temperature), float(sp.top_p), float(sp.min_p), float(sp.repetition_penalty), float(sp.presence_penalty),
              float(sp.frequency_penalty)] + [float(v) for v in lb.values()]
    return ints, floats


def _sampling_from_wire(ints, floats):
    from ..runtime.engine import SamplingParams
    nb = ints[2]
    lb = {ints[3 + i]: floats[6 + i] for i in range(nb)} or None
    return SamplingParams(temperature=floats[0], top_k=ints[0], top_p=floats[1], min_p=floats[2], max_tokens=ints[1],
                          repetition_penalty=floats[3], presence_penalty=floats[4], frequency_penalty=floats[5], logit_bias=lb)


class TpLeaderEngine:
    """Rank 0's engine as seen by ``ServingEngine``: every call is announced to the followers, then run locally."""

    def __init__(self, engine, group, comm=None):
        self.engine, self.chan, self.comm = engine, _Channel(group), comm
        self.cfg, self.num_pages = engine.cfg, engine.num_pages

    # attributes the serving layer reads
    @property
    def slots(self):
        return self.engine.slots

    @property
    def gemm_ok(self):
        return self.engine.gemm_ok

    @property
    def mcfg(self):
        return self.engine.mcfg

    def free_slots(self):
        return self.engine.free_slots()

    def open_slot(self, slot: int, reserve: int):
        self.chan.send(OP_OPEN, slot, [reserve])
        return self.engine.open_slot(slot, reserve)

    def close_slot(self, slot: int) -> None:
        self.chan.send(OP_CLOSE, slot)
        self.engine.close_slot(slot)

    def set_sampling(self, slot: int, sp) -> None:
        self.chan.send(OP_SAMPLING, slot, *_sampling_to_wire(sp))
        self.engine.set_sampling(slot, sp)

    def set_token_mask(self, slot: int, allowed) -> None:
        if allowed is None:
            self.chan.send(OP_MASK, slot, [0])
        else:
            bits = np.packbits(np.asarray(allowed, dtype=bool))
            self.chan.send(OP_MASK, slot, [1, len(allowed)] + [int(b) for b in bits])
        self.engine.set_token_mask(slot, allowed)

    def prefill(self, slot: int, tokens: Sequence[int]) -> int:
        self.chan.send(OP_PREFILL, slot, [int(t) for t in tokens])
        return self.engine.prefill(slot, tokens)

    def feed(self, slot_tokens: Dict[int, int]):
        flat: List[int] = []
        for s, t in slot_tokens.items():
            flat += [int(s), int(t)]
        self.chan.send(OP_FEED, -1, flat)
        return self.engine.feed(slot_tokens)

    def score_tokens(self, tokens: Sequence[int], want_embedding: bool = False, top_k: int = 0) -> dict:
        self.chan.send(OP_SCORE, 1 if want_embedding else 0, [int(t) for t in tokens])
        return self.engine.score_tokens(tokens, want_embedding=want_embedding, top_k=0)

    def draft_step(self, slot: int, token: int, layers: Sequence[int]) -> int:
        self.chan.send(OP_DRAFT, slot, [int(token)] + [int(l) for l in layers])
        return self.engine.draft_step(slot, token, layers)

    def forward_tokens(self, slot: int, tokens: Sequence[int]) -> List[int]:
        self.chan.send(OP_FORWARD, slot, [int(t) for t in tokens])
        return self.engine.forward_tokens(slot, tokens)

    def rollback(self, slot: int, position: int) -> None:
        self.chan.send(OP_ROLLBACK, slot, [position])
        self.engine.rollback(slot, position)

    def reset(self) -> None:
        """After a failed step: every rank returns its engine to the post-load state (the followers ignore the commands that
        were sent between their failure and this one, see ``follower_loop``).  Raises when this rank's device does not answer."""
        self.chan.send(OP_RESET)
        self.engine.reset()

    def shutdown(self, leave: bool = True) -> None:
        """Release the followers (they leave ``follower_loop``).  With ``leave`` (servers) this rank then takes its engine
        and the process group down in order - captured graphs first, then the peer-memory mappings, then the group - as the
        followers do after their loop."""
        self.chan.send(OP_STOP)
        if leave:
            leave_group(self.engine, self.comm)


def leave_group(engine, comm) -> None:
    """Orderly exit of one tensor-parallel serving rank (every rank calls it)."""
    if hasattr(engine, "close"):
        engine.close()
    if comm is not None:
        comm.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def follower_loop(engine, group) -> int:
    """Execute rank 0's engine calls until it sends the stop command.  Returns the number of calls executed.
    A call that raises here (the same status word or CUDA error that stops rank 0's loop) does not end the follower: it stops
    executing commands - the sequence state is no longer in step with rank 0 - until rank 0 sends the reset command, resets its
    engine and goes on; if the reset itself raises, the device is lost and the exception ends this rank."""
    chan, n, failed = _Channel(group), 0, None
    while True:
        op, slot, ints, floats = chan.recv()
        if op == OP_STOP:
            return n
        if op == OP_RESET:
            engine.reset()
            failed = None
            continue
        if failed is not None:
            continue
        n += 1
        try:
            _execute(engine, op, slot, ints, floats)
        except Exception as e:                              # noqa: BLE001 - reported, then wait for the reset
            failed = repr(e)
            log.error("tensor-parallel follower: engine call %d failed (%s); waiting for a reset", op, failed)


def _execute(engine, op, slot, ints, floats) -> None:
    if op == OP_OPEN:
        engine.open_slot(slot, ints[0])
    elif op == OP_CLOSE:
        engine.close_slot(slot)
    elif op == OP_SAMPLING:
        engine.set_sampling(slot, _sampling_from_wire(ints, floats))
    elif op == OP_MASK:
        engine.set_token_mask(slot, None if ints[0] == 0 else np.unpackbits(np.asarray(ints[2:], dtype=np.uint8))[: ints[1]].astype(bool))
    elif op == OP_PREFILL:
        engine.prefill(slot, ints)
    elif op == OP_FEED:
        engine.feed({ints[i]: ints[i + 1] for i in range(0, len(ints), 2)})
    elif op == OP_SCORE:
        engine.score_tokens(ints, want_embedding=bool(slot))
    elif op == OP_DRAFT:
        engine.draft_step(slot, ints[0], ints[1:])
    elif op == OP_FORWARD:
        engine.forward_tokens(slot, ints)
    elif op == OP_ROLLBACK:
        engine.rollback(slot, ints[0])
    else:
        raise RuntimeError(f"unknown tensor-parallel serving command {op}")


def init_tp(mode: str = "fused"):
    """Process-group set-up of one tensor-parallel serving rank (launched by ``torch.distributed.run``): returns
    ``(rank, world, device, comm, command_group)``."""
    import os
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from .tp import make_tp_comm
    comm = make_tp_comm(rank, world, dev, mode=mode)
    group = dist.new_group(backend="gloo")
    return rank, world, dev, comm, group
