"""Blocking tensor/sequence-parallel collectives and their autograd maps (legacy synchronous
path, used by `Trainer` and by tests as the simplest correct TP/SP implementation).

Conjugate pairs (reference: `src/sharded_runtime/parallel/mappings.py:12-148`,
`docs/tp_sp_contracts.md`): `copy_to_tp` (identity / all-reduce) with `reduce_from_tp`
(all-reduce / identity) for plain TP, and `gather_sequence` (all-gather / reduce-scatter) with
`reduce_scatter_sequence` (reduce-scatter / all-gather) for sequence parallelism.  On gloo the
reduce-scatter is computed as all-reduce + slice: same numbers, different cost.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd.function import once_differentiable


@dataclass(frozen=True)
class TPGroup:
    process_group: Any = None
    degree: int = 1
    rank: int = 0
    backend: str = "local"

    def __post_init__(self) -> None:
        if self.degree < 1 or not 0 <= self.rank < self.degree:
            raise ValueError("Invalid TP group degree/rank")
        if self.degree > 1 and self.process_group is None:
            raise ValueError("A non-singleton TP group requires an explicit ProcessGroup")

    @classmethod
    def from_process_group(cls, group: Any = None) -> "TPGroup":
        if not dist.is_initialized():
            if group is not None:
                raise ValueError("ProcessGroup supplied before distributed initialization")
            return cls()
        if group is None:
            raise ValueError("Pass the explicit TP ProcessGroup; WORLD is not an implicit TP group")
        return cls(group, dist.get_world_size(group), dist.get_rank(group), str(dist.get_backend(group)))

    def sum(self, x: Tensor) -> Tensor:
        if self.degree == 1:
            return x
        out = x.contiguous().clone()  # never mutate an upstream (possibly shared) gradient
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.process_group)
        return out

    def gather(self, x: Tensor, dim: int) -> Tensor:
        if self.degree == 1:
            return x
        mine = x.contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.degree)]
        dist.all_gather(parts, mine, group=self.process_group)
        return torch.cat(parts, dim=dim)

    def sequence_shard(self, x: Tensor) -> Tensor:
        if x.ndim < 2 or x.shape[1] % self.degree:
            raise ValueError("Sequence length must be divisible by the TP degree")
        width = x.shape[1] // self.degree
        return x.narrow(1, self.rank * width, width)

    def reduce_scatter_sequence(self, x: Tensor) -> Tensor:
        if x.ndim != 3 or x.shape[1] == 0 or x.shape[1] % self.degree:
            raise ValueError("SP ReduceScatter requires a divisible full sequence in [B,S,H]")
        if self.degree == 1:
            return x
        if self.backend == "gloo":
            return self.sequence_shard(self.sum(x)).clone()
        if self.backend != "nccl":
            raise ValueError(f"Unsupported TP backend: {self.backend}")
        packed = x.movedim(1, 0).contiguous()
        out = packed.new_empty((packed.shape[0] // self.degree, *packed.shape[1:]))
        dist.reduce_scatter_tensor(out, packed, op=dist.ReduceOp.SUM, group=self.process_group)
        return out.movedim(0, 1).contiguous()

    def broadcast(self, x: Tensor) -> None:
        if self.degree > 1:
            dist.broadcast(x, src=dist.get_global_rank(self.process_group, 0), group=self.process_group)


def _map(name, forward, backward):
    """Build an autograd Function from a (forward, backward) pair of group methods."""

    class Map(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, group):  # noqa: D401
            ctx.group = group
            return forward(group, x)

        @staticmethod
        @once_differentiable
        def backward(ctx, grad):
            return backward(ctx.group, grad), None

    Map.__name__ = Map.__qualname__ = name
    return Map


def _identity(group, x):
    return x.view_as(x)


def _gather_checked(group, x):
    if x.ndim != 3 or x.shape[1] == 0:
        raise ValueError("SP AllGather expects nonempty sequence shards in [B,S_local,H]")
    return group.gather(x, dim=1)


_CopyToTP = _map("_CopyToTP", _identity, lambda g, t: g.sum(t))
# the output adjoint is replicated on every TP rank, so backward must not count it T times
_ReduceFromTP = _map("_ReduceFromTP", lambda g, t: g.sum(t), lambda g, t: t)
_GatherSequence = _map("_GatherSequence", _gather_checked, lambda g, t: g.reduce_scatter_sequence(t))
_ReduceScatterSequence = _map("_ReduceScatterSequence", lambda g, t: g.reduce_scatter_sequence(t),
                              lambda g, t: g.gather(t, dim=1))


def copy_to_tp(x: Tensor, group: TPGroup) -> Tensor:
    return _CopyToTP.apply(x, group)


def reduce_from_tp(x: Tensor, group: TPGroup) -> Tensor:
    return _ReduceFromTP.apply(x, group)


def gather_sequence(x: Tensor, group: TPGroup) -> Tensor:
    return _GatherSequence.apply(x, group)


def reduce_scatter_sequence(x: Tensor, group: TPGroup) -> Tensor:
    return _ReduceScatterSequence.apply(x, group)
