"""Portable (torch-op) parameter consumers of the Qwen2 units.

These are the autograd functions the runtime-driven forward uses on CPU/gloo and on the NCCL
baseline path.  Shared rules (reference: `src/sharded_runtime/runtime/qwen2_operators.py:11-204`):

* a consumer never saves a full parameter for backward: it saves only its *compact local* input
  and re-reads the weight of the unit's current generation in backward (`handle.weight()`);
* column projections that read the same input share one sequence all-gather (q/k/v; gate/up);
  backward re-gathers the local input once, forms every branch's dW, sums the branches' dX in
  FP32 and issues one sequence reduce-scatter;
* row projections reduce-scatter their partial output over the sequence (all-reduce without SP,
  nothing for a TP-replicated weight such as the LM head);
* GEMMs run in the runtime's compute dtype in forward *and* backward, parameter gradients are
  returned in the master dtype (FP32).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch.autograd.function import once_differentiable
from torch.nn import functional as F


def compact(x):
    """Contiguous tensor that owns exactly its elements (no oversized storage kept alive)."""
    value = x.contiguous()
    if value.untyped_storage().nbytes() != value.numel() * value.element_size():
        value = value.clone()
    return value


@dataclass
class Branch:
    """One projection of a column group: weight (and bias) handle of the owning unit."""

    weight: object
    bias: object = None


class ColumnProjection(torch.autograd.Function):
    """N column-parallel linears on one (sequence-gathered) input."""

    @staticmethod
    def forward(ctx, x, runtime, branches, boundary, *weights):
        ctx.set_materialize_grads(False)
        tp, sp = runtime.tp, runtime.sp
        ctx.runtime, ctx.branches, ctx.boundary, ctx.input_dtype = runtime, branches, boundary, x.dtype
        unit = branches[0].weight.unit
        unit.annotate("FWD")
        local = compact(x.to(runtime.compute_dtype))
        ctx.save_for_backward(local)
        ctx.local_lease = runtime.comm.buffer(local, "projection_local_saved")
        pending = tp.issue_gather(local, 1) if sp else None
        # a deferred parameter prefetch goes between the gather's issue and its consumption
        unit.prefetch_after_input(boundary, "FWD")
        source = tp.finish_gather(pending) if pending is not None else local
        outputs, cursor = [], 0
        for branch in branches:
            w = weights[cursor].to(source.dtype)
            b = weights[cursor + 1].to(source.dtype) if branch.bias is not None else None
            outputs.append(F.linear(source, w, b))
            cursor += 2 if branch.bias is not None else 1
        if pending is not None:
            tp.retire_activation(source)
        return tuple(outputs)

    @staticmethod
    @once_differentiable
    def backward(ctx, *grads):
        runtime = ctx.runtime
        tp, sp = runtime.tp, runtime.sp
        unit = ctx.branches[0].weight.unit
        unit.annotate("BWD")
        (local,) = ctx.saved_tensors
        source = tp.gather(local, 1) if sp else local
        flat = source.reshape(-1, source.shape[-1])
        dparams, dx = [], None
        for grad, branch in zip(grads, ctx.branches):
            if grad is None:
                raise RuntimeError("Unused Qwen projection branches are unsupported")
            weight = branch.weight.weight()
            g = grad.to(local.dtype)
            g2 = g.reshape(-1, g.shape[-1])
            dparams.append((g2.t() @ flat).to(weight.dtype))
            part = (g @ weight.to(local.dtype)).to(torch.float32)
            dx = part if dx is None else dx + part
            if branch.bias is not None:
                dparams.append(grad.float().sum(tuple(range(grad.ndim - 1))).to(weight.dtype))
        if sp:
            tp.retire_activation(source)
            dx = tp.reduce_scatter_sequence(dx)
        elif tp.degree > 1:
            dx = tp.sum(dx)
        runtime.comm.retire(ctx.local_lease)
        return (dx.to(ctx.input_dtype), None, None, None, *dparams)


class RowLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, runtime, handle, replicated):
        tp, sp = runtime.tp, runtime.sp
        handle.unit.annotate("FWD")
        ctx.runtime, ctx.handle, ctx.replicated, ctx.input_dtype = runtime, handle, replicated, x.dtype
        local = compact(x.to(runtime.compute_dtype))
        ctx.save_for_backward(local)
        handle.unit.prefetch_after_input(handle, "FWD")
        partial = F.linear(local, weight.to(local.dtype))
        if replicated or tp.degree == 1:
            return partial
        return tp.reduce_scatter_sequence(partial) if sp else tp.sum(partial)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        runtime, handle = ctx.runtime, ctx.handle
        tp, sp = runtime.tp, runtime.sp
        handle.unit.annotate("BWD")
        (local,) = ctx.saved_tensors
        g = compact(grad)
        gathered = sp and not ctx.replicated and tp.degree > 1
        if gathered:
            g = tp.gather(g, 1)
        handle.unit.prefetch_after_input(handle, "BWD")
        weight = handle.weight()
        gc = g.to(local.dtype)
        dw = gc.reshape(-1, gc.shape[-1]).t() @ local.reshape(-1, local.shape[-1])
        dx = gc @ weight.to(local.dtype)
        if gathered:
            tp.retire_activation(g)
        return dx.to(ctx.input_dtype), dw.to(weight.dtype), None, None, None


class NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, handle, eps):
        handle.unit.annotate("FWD")
        ctx.handle, ctx.input_dtype = handle, x.dtype
        wide = compact(x.float())
        inv = torch.rsqrt(wide.square().mean(-1, keepdim=True) + eps)
        normalized = (wide * inv).to(x.dtype)
        ctx.save_for_backward(wide, inv, normalized)
        out = normalized * weight
        handle.unit.prefetch_after_input(handle, "FWD")
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        handle = ctx.handle
        handle.unit.annotate("BWD")
        wide, inv, normalized = ctx.saved_tensors
        weight = handle.weight()
        handle.unit.prefetch_after_input(handle, "BWD")
        scaled = grad.float() * weight.float()
        dx = inv * (scaled - wide * inv.square() * (scaled * wide).mean(-1, keepdim=True))
        dw = (grad.float() * normalized.float()).sum(tuple(range(grad.ndim - 1)))
        return dx.to(ctx.input_dtype), dw.to(weight.dtype), None, None


class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, handle, padding_idx):
        ctx.handle, ctx.padding_idx = handle, padding_idx
        ctx.save_for_backward(ids)
        out = F.embedding(ids, weight, padding_idx=padding_idx)
        handle.unit.prefetch_after_input(handle, "FWD")
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        handle = ctx.handle
        handle.unit.annotate("BWD")
        (ids,) = ctx.saved_tensors
        # the adjoint needs only the shape, never the forward's full parameter
        dw = torch.zeros(handle.spec.tp_local_shape, device=grad.device, dtype=handle.spec.dtype)
        dw.index_add_(0, ids.reshape(-1), grad.reshape(-1, grad.shape[-1]).to(dw.dtype))
        if ctx.padding_idx is not None:
            dw[ctx.padding_idx].zero_()
        return None, dw, None, None
