"""Parallelism configuration and rank arithmetic: tensor / pipeline / data parallel sizes,
shard shapes, pipeline stage partitioning and bubble ratio, ZeRO-inference offload settings,
and a single-process mock communicator for rank-math tests.

Capability parity with the reference's ``parallel`` module (``ParallelConfig``,
``TensorParallel``, ``PipelineParallel``, ``ZeroOffload``, ``DistributedContext`` and the mock
``Communicator``: src/parallel/mod.rs:79-376, src/parallel/mod_all_reduce_communicator.rs:2-436,
src/parallel/distributed_context_impl.rs:4-97).  The real node-local communicators live in
``realizar_b200.parallel.tp``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


class ParallelError(ValueError):
    pass


@dataclass(frozen=True)
class ParallelConfig:
    """world = tp * pp * dp; the tensor-parallel index varies fastest, then pipeline, then data."""
    tp_size: int = 1
    pp_size: int = 1
    dp_size: int = 1
    rank: int = 0

    def __post_init__(self):
        if min(self.tp_size, self.pp_size, self.dp_size) < 1:
            raise ParallelError("parallel sizes must be >= 1")
        if not 0 <= self.rank < self.world_size:
            raise ParallelError(f"rank {self.rank} out of range for world size {self.world_size}")

    @property
    def world_size(self) -> int: return self.tp_size * self.pp_size * self.dp_size
    @property
    def tp_rank(self) -> int: return self.rank % self.tp_size
    @property
    def pp_rank(self) -> int: return (self.rank // self.tp_size) % self.pp_size
    @property
    def dp_rank(self) -> int: return self.rank // (self.tp_size * self.pp_size)
    @property
    def is_distributed(self) -> bool: return self.world_size > 1

    def tp_group(self) -> List[int]:
        base = self.rank - self.tp_rank
        return list(range(base, base + self.tp_size))


class ReduceOp:
    SUM, AVG, MAX, MIN = "sum", "avg", "max", "min"


class MockCommunicator:
    """Single-process stand-in: every rank holds the same tensor, so ``all_reduce(SUM)`` multiplies
    by the world size, AVG / MAX / MIN are the identity, ``all_gather`` repeats along dim 0 and
    ``reduce_scatter`` keeps this rank's chunk of the (world-times) sum."""

    def __init__(self, world_size: int = 1, rank: int = 0):
        if world_size < 1 or not 0 <= rank < world_size:
            raise ParallelError("invalid communicator geometry")
        self.world_size, self.rank = world_size, rank
        self.calls: List[str] = []

    def all_reduce(self, t: torch.Tensor, op: str = ReduceOp.SUM) -> torch.Tensor:
        self.calls.append(f"all_reduce:{op}")
        return t * self.world_size if op == ReduceOp.SUM else t.clone()

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        self.calls.append("all_gather")
        return torch.cat([t] * self.world_size, dim=0)

    def reduce_scatter(self, t: torch.Tensor, op: str = ReduceOp.SUM) -> torch.Tensor:
        self.calls.append(f"reduce_scatter:{op}")
        if t.shape[0] % self.world_size:
            raise ParallelError("reduce_scatter needs dim 0 divisible by the world size")
        chunk = t.shape[0] // self.world_size
        out = t[self.rank * chunk:(self.rank + 1) * chunk]
        return out * self.world_size if op == ReduceOp.SUM else out.clone()

    def barrier(self) -> None:
        self.calls.append("barrier")


class TorchCommunicator:
    """The same interface over a ``torch.distributed`` process group (gloo on CPU, NCCL on GPU)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world_size, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def all_reduce(self, t, op: str = ReduceOp.SUM):
        d = self.dist
        out = t.clone()
        d.all_reduce(out, op={ReduceOp.SUM: d.ReduceOp.SUM, ReduceOp.AVG: d.ReduceOp.SUM, ReduceOp.MAX: d.ReduceOp.MAX, ReduceOp.MIN: d.ReduceOp.MIN}[op], group=self.group)
        return out / self.world_size if op == ReduceOp.AVG else out

    def all_gather(self, t):
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        self.dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    def reduce_scatter(self, t, op: str = ReduceOp.SUM):
        full = self.all_reduce(t, op)
        chunk = t.shape[0] // self.world_size
        return full[self.rank * chunk:(self.rank + 1) * chunk].clone()

    def barrier(self):
        self.dist.barrier(group=self.group)


class TensorParallel:
    """Megatron-style linear layers over a communicator: column-parallel shards the output
    features (no communication), row-parallel shards the input features and all-reduces; the
    bias of a row-parallel layer is added on rank 0 only so it is counted once."""

    def __init__(self, size: int, rank: int, comm=None):
        if size < 1 or not 0 <= rank < size:
            raise ParallelError("invalid tensor-parallel geometry")
        self.size, self.rank = size, rank
        self.comm = comm or MockCommunicator(size, rank)

    def shard_range(self, dim: int) -> Tuple[int, int]:
        if dim % self.size:
            raise ParallelError(f"dimension {dim} is not divisible by the tensor-parallel size {self.size}")
        c = dim // self.size
        return self.rank * c, (self.rank + 1) * c

    def shard_columns(self, weight: torch.Tensor) -> torch.Tensor:
        """``weight [out, in]`` -> rows of this rank's output features."""
        a, b = self.shard_range(weight.shape[0])
        return weight[a:b]

    def shard_rows(self, weight: torch.Tensor) -> torch.Tensor:
        """``weight [out, in]`` -> this rank's slice of the input features."""
        a, b = self.shard_range(weight.shape[1])
        return weight[:, a:b]

    def column_parallel_linear(self, x, weight_shard, bias_shard=None):
        y = x @ weight_shard.T
        return y + bias_shard if bias_shard is not None else y

    def row_parallel_linear(self, x_shard, weight_shard, bias=None):
        y = x_shard @ weight_shard.T
        if bias is not None and self.rank == 0:
            y = y + bias
        return self.comm.all_reduce(y, ReduceOp.SUM)


@dataclass
class PipelineStats:
    num_stages: int
    num_micro_batches: int
    bubble_ratio: float
    layers_per_stage: List[int]


class PipelineParallel:
    """GPipe-style stage partitioning: contiguous layer ranges (earlier stages take the remainder),
    micro-batch size and the bubble ratio (pp - 1) / (pp + m - 1)."""

    def __init__(self, num_stages: int, stage: int, num_layers: int, num_micro_batches: int = 1):
        if num_stages < 1 or not 0 <= stage < num_stages or num_layers < num_stages or num_micro_batches < 1:
            raise ParallelError("invalid pipeline geometry")
        self.num_stages, self.stage, self.num_layers, self.num_micro_batches = num_stages, stage, num_layers, num_micro_batches

    def layer_range(self, stage: Optional[int] = None) -> Tuple[int, int]:
        s = self.stage if stage is None else stage
        base, rem = divmod(self.num_layers, self.num_stages)
        start = s * base + min(s, rem)
        return start, start + base + (1 if s < rem else 0)

    def micro_batch_size(self, batch: int) -> int:
        return -(-batch // self.num_micro_batches)

    @property
    def bubble_ratio(self) -> float:
        return (self.num_stages - 1) / (self.num_stages + self.num_micro_batches - 1)

    @property
    def is_first(self) -> bool: return self.stage == 0
    @property
    def is_last(self) -> bool: return self.stage == self.num_stages - 1

    def stats(self) -> PipelineStats:
        return PipelineStats(self.num_stages, self.num_micro_batches, self.bubble_ratio,
                             [self.layer_range(s)[1] - self.layer_range(s)[0] for s in range(self.num_stages)])


@dataclass(frozen=True)
class ZeroOffload:
    """ZeRO-inference style placement switches and the resulting GPU-memory saving estimate."""
    offload_params: bool = False
    offload_kv: bool = False
    pin_memory: bool = True
    param_fraction_on_gpu: float = 1.0

    def memory_savings_ratio(self) -> float:
        r = 0.0
        if self.offload_params:
            r += 0.7 * (1.0 - self.param_fraction_on_gpu)
        if self.offload_kv:
            r += 0.2
        return min(r, 0.95)


@dataclass
class DistributedContext:
    config: ParallelConfig
    tp: Optional[TensorParallel] = None
    pp: Optional[PipelineParallel] = None
    zero: ZeroOffload = field(default_factory=ZeroOffload)

    @classmethod
    def create(cls, tp=1, pp=1, dp=1, rank=0, num_layers: int = 0, micro_batches: int = 1, comm=None) -> "DistributedContext":
        cfg = ParallelConfig(tp, pp, dp, rank)
        t = TensorParallel(tp, cfg.tp_rank, comm) if tp > 1 else None
        p = PipelineParallel(pp, cfg.pp_rank, num_layers, micro_batches) if pp > 1 else None
        return cls(cfg, t, p)

    @property
    def is_distributed(self) -> bool:
        return self.config.is_distributed
