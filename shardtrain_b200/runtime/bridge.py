"""Autograd bridge between the persistent shard leaves and the materialised full parameters.

`UnitMaterialize` is one multi-output node per unit: forward finishes the (possibly prefetched)
materialisation and returns the full parameters; autograd runs its backward exactly once, after
every consumer of the unit has produced its weight gradient, and that is where the unit's
gradient reduce-scatter is issued.  `PreBackward` is an identity on the unit's output whose
backward fires *before* the unit's consumers run backward, which is where the unit is
re-materialised (reference: `src/sharded_runtime/runtime/bridge.py:9-47`).

The reduced shard gradients are committed into the persistent gradient arena by the unit itself
(`UnitState.reduce`), so this node returns no gradient for the shard leaves.
"""

from __future__ import annotations

import torch
from torch.autograd.function import once_differentiable


class UnitMaterialize(torch.autograd.Function):
    @staticmethod
    def forward(ctx, unit, *shards):
        ctx.unit = unit
        ctx.set_materialize_grads(False)
        comm = unit.runtime.comm
        # copy-out always runs on the compute stream, whichever stream owns this graph node
        with comm.stream_context("compute"):
            outputs = unit.runtime.materializer.finish(unit)
        # (None: the materialiser left the wait to the first reader of the gathered parameters)
        if comm.streams and unit.lease.copy_out_ready_event is not None:
            comm.wait_event(unit.lease.copy_out_ready_event, dependency_type="DATA_DEP",
                            consumer="materialize_outputs")
        return outputs

    @staticmethod
    @once_differentiable
    def backward(ctx, *grads):
        unit = ctx.unit
        unit.annotate("BWD")
        comm = unit.runtime.comm
        if comm.streams and comm.diagnostics_enabled:
            comm.event("bridge_backward_stream",
                       cuda_stream=unit.runtime.comm.current_stream().cuda_stream)
        unit.reduce(grads)
        return (None,) * (1 + len(unit.handles))


class PreBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, output, unit):
        ctx.unit = unit
        return output.view_as(output)

    @staticmethod
    @once_differentiable
    def backward(ctx, gradient):
        ctx.unit.pre_backward()
        return gradient, None
