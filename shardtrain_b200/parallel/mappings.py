"""Blocking tensor/sequence-parallel collectives and their autograd maps (legacy synchronous
path, used by `Trainer` and by tests as the simplest correct TP/SP implementation).

Every map of Megatron-style TP/SP is one of four collectives in the forward and its conjugate
in the backward (`docs/tp_sp_contracts.md`, `src/sharded_runtime/parallel/mappings.py:12-148` of
the reference):

    name                      forward                  backward
    copy_to_tp                identity                 all-reduce
    reduce_from_tp            all-reduce               identity
    gather_sequence           all-gather (seq)         reduce-scatter (seq)
    reduce_scatter_sequence   reduce-scatter (seq)     all-gather (seq)

The table below is the whole definition: one autograd Function looks the pair up by name.  The
collectives themselves are small functions over a `TPGroup`; on gloo the sequence
reduce-scatter is computed as all-reduce + slice (same numbers, different cost).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd.function import once_differentiable


@dataclass(frozen=True)
class TPGroup:
    """A tensor-parallel communicator with its size, this rank's index and its backend name."""

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

    @property
    def alone(self) -> bool:
        return self.degree == 1

    # the collectives, as methods for callers that hold a group
    def sum(self, x: Tensor) -> Tensor:
        return all_reduce_sum(x, self)

    def gather(self, x: Tensor, dim: int) -> Tensor:
        return all_gather_cat(x, self, dim)

    def sequence_shard(self, x: Tensor) -> Tensor:
        return own_sequence_slice(x, self)

    def reduce_scatter_sequence(self, x: Tensor) -> Tensor:
        return reduce_scatter_seq(x, self)

    def broadcast(self, x: Tensor) -> None:
        if not self.alone:
            root = dist.get_global_rank(self.process_group, 0)
            dist.broadcast(x, src=root, group=self.process_group)


# ---------------------------------------------------------------------------- collectives
def all_reduce_sum(x: Tensor, group: TPGroup) -> Tensor:
    """Out-of-place SUM: the input may be an upstream gradient shared with other consumers."""
    if group.alone:
        return x
    total = x.contiguous().clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group.process_group)
    return total


def all_gather_cat(x: Tensor, group: TPGroup, dim: int) -> Tensor:
    if group.alone:
        return x
    piece = x.contiguous()
    pieces = [torch.empty_like(piece) for _ in range(group.degree)]
    dist.all_gather(pieces, piece, group=group.process_group)
    return torch.cat(pieces, dim=dim)


def own_sequence_slice(x: Tensor, group: TPGroup) -> Tensor:
    if x.ndim < 2 or x.shape[1] % group.degree:
        raise ValueError("Sequence length must be divisible by the TP degree")
    width = x.shape[1] // group.degree
    return x.narrow(1, group.rank * width, width)


def _reduce_scatter_by_all_reduce(x: Tensor, group: TPGroup) -> Tensor:
    return own_sequence_slice(all_reduce_sum(x, group), group).clone()


def _reduce_scatter_native(x: Tensor, group: TPGroup) -> Tensor:
    # reduce_scatter_tensor splits dimension 0: put the sequence first, and back afterwards
    sequence_major = x.movedim(1, 0).contiguous()
    mine = sequence_major.new_empty((sequence_major.shape[0] // group.degree, *sequence_major.shape[1:]))
    dist.reduce_scatter_tensor(mine, sequence_major, op=dist.ReduceOp.SUM, group=group.process_group)
    return mine.movedim(0, 1).contiguous()


_REDUCE_SCATTER_BY_BACKEND: dict[str, Callable[[Tensor, TPGroup], Tensor]] = {
    "gloo": _reduce_scatter_by_all_reduce,
    "nccl": _reduce_scatter_native,
}


def reduce_scatter_seq(x: Tensor, group: TPGroup) -> Tensor:
    if x.ndim != 3 or x.shape[1] == 0 or x.shape[1] % group.degree:
        raise ValueError("SP ReduceScatter requires a divisible full sequence in [B,S,H]")
    if group.alone:
        return x
    try:
        implementation = _REDUCE_SCATTER_BY_BACKEND[group.backend]
    except KeyError:
        raise ValueError(f"Unsupported TP backend: {group.backend}") from None
    return implementation(x, group)


def _gather_seq(x: Tensor, group: TPGroup) -> Tensor:
    if x.ndim != 3 or x.shape[1] == 0:
        raise ValueError("SP AllGather expects nonempty sequence shards in [B,S_local,H]")
    return all_gather_cat(x, group, dim=1)


def _same(x: Tensor, group: TPGroup) -> Tensor:
    return x.view_as(x)          # a new tensor object, so autograd records the node


# name -> (forward collective, backward collective).  reduce_from_tp's adjoint is the identity:
# the output gradient is already replicated on every TP rank and must not be counted T times.
CONJUGATE_PAIRS: dict[str, tuple[Callable, Callable]] = {
    "copy_to_tp": (_same, all_reduce_sum),
    "reduce_from_tp": (all_reduce_sum, lambda g, group: g),
    "gather_sequence": (_gather_seq, reduce_scatter_seq),
    "reduce_scatter_sequence": (reduce_scatter_seq, lambda g, group: all_gather_cat(g, group, dim=1)),
}


class _ConjugateMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, group: TPGroup, name: str) -> Tensor:
        ctx.group, ctx.name = group, name
        return CONJUGATE_PAIRS[name][0](x, group)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad: Tensor):
        return CONJUGATE_PAIRS[ctx.name][1](grad, ctx.group), None, None


def copy_to_tp(x: Tensor, group: TPGroup) -> Tensor:
    return _ConjugateMap.apply(x, group, "copy_to_tp")


def reduce_from_tp(x: Tensor, group: TPGroup) -> Tensor:
    return _ConjugateMap.apply(x, group, "reduce_from_tp")


def gather_sequence(x: Tensor, group: TPGroup) -> Tensor:
    return _ConjugateMap.apply(x, group, "gather_sequence")


def reduce_scatter_sequence(x: Tensor, group: TPGroup) -> Tensor:
    return _ConjugateMap.apply(x, group, "reduce_scatter_sequence")
