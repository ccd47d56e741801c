"""Bias-free column / row parallel linears of the legacy synchronous path
(`src/sharded_runtime/parallel/tp_linear.py:17-87`).  A column linear keeps rows
[rank*out/T, (rank+1)*out/T) of the `[out, in]` weight, a row linear the matching columns."""

from __future__ import annotations

from torch import Tensor, nn
from torch.nn import functional as F

from shardtrain_b200.parallel.mappings import (
    TPGroup, copy_to_tp, gather_sequence, reduce_from_tp, reduce_scatter_sequence,
)
from shardtrain_b200.runtime.qwen2_adapter import ParameterPartition

__all__ = ["ParameterPartition", "ColumnParallelLinear", "RowParallelLinear"]


def _check(linear: nn.Linear, degree: int, dim: int) -> None:
    if type(linear) is not nn.Linear or linear.bias is not None:
        raise ValueError("M1 TP Linear requires an ordinary bias-free nn.Linear")
    if linear.weight.shape[dim] % degree:
        raise ValueError("TP partition dimension must be divisible by TP degree")


class _ParallelLinear(nn.Module):
    split_dim = 0

    def __init__(self, linear: nn.Linear, group: TPGroup, *, sp: bool = False) -> None:
        super().__init__()
        _check(linear, group.degree, self.split_dim)
        self.group, self.sp = group, sp
        self.partition = ParameterPartition(tuple(linear.weight.shape), self.split_dim,
                                            group.rank, group.degree)
        self.weight = nn.Parameter(self.partition.local_slice(linear.weight).detach().clone())
        self.out_features, self.in_features = self.weight.shape


class ColumnParallelLinear(_ParallelLinear):
    split_dim = 0

    def forward(self, x: Tensor) -> Tensor:
        source = gather_sequence(x, self.group) if self.sp else copy_to_tp(x, self.group)
        return F.linear(source, self.weight)


class RowParallelLinear(_ParallelLinear):
    split_dim = 1

    def forward(self, x: Tensor) -> Tensor:
        partial = F.linear(x, self.weight)
        if self.sp:
            return reduce_scatter_sequence(partial, self.group)
        return reduce_from_tp(partial, self.group)
