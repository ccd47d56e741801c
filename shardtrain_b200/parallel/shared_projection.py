"""One sequence all-gather feeding several column projections (q/k/v, gate/up).

Forward gathers the compact local input once and applies every projection; backward re-gathers
that local input once, forms each branch's dW, sums the branches' dX and reduce-scatters the sum
once.  Only the local shard is saved (`src/sharded_runtime/parallel/shared_projection.py:26-111`).
"""

from __future__ import annotations

import torch
from torch.autograd.function import once_differentiable
from torch.nn import functional as F


class SharedProjection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, *weights):
        if not all(w.requires_grad for w in weights):
            raise RuntimeError("Shared projections require every weight to be trainable")
        ctx.set_materialize_grads(False)
        ctx.group = group
        local = x.contiguous()
        ctx.save_for_backward(local, *weights)
        source = group.gather(local, 1)
        return tuple(F.linear(source, w) for w in weights)

    @staticmethod
    @once_differentiable
    def backward(ctx, *grads):
        if any(g is None for g in grads):
            raise RuntimeError("Unused shared-projection branches are unsupported")
        local, *weights = ctx.saved_tensors
        source = ctx.group.gather(local, 1)
        flat = source.reshape(-1, source.shape[-1])
        dweights, dx = [], None
        for g, w in zip(grads, weights):
            g = g.contiguous()
            dweights.append(g.reshape(-1, g.shape[-1]).t() @ flat)
            part = g @ w
            dx = part if dx is None else dx + part
        dx = ctx.group.reduce_scatter_sequence(dx)
        return (dx if ctx.needs_input_grad[0] else None, None, *dweights)


class SharedProjectionGroup:
    """Callable that replaces the separate projection calls of a block; the projection modules
    keep owning their parameters."""

    def __init__(self, projections, group, role):
        self.projections, self.group, self.role = tuple(projections), group, role

    def __call__(self, x):
        return SharedProjection.apply(x, self.group, *(p.weight for p in self.projections))
