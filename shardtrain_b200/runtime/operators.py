"""Sharded-runtime registration of the toy block model (`TransformerBlock` or a `Sequential`).

Every block becomes one unit of nine parameters.  After registration the module tree still yields
the original names (`{i}.attention.q_proj.weight`, ...) but each parameter is the rank's flat
FP32 shard, and each block's `forward` is driven by the runtime with materialised weights through
the same portable consumers as the Qwen path (`ColumnProjection`, `RowLinear`, `NormFn`), so the
lifecycle rules (one forward / backward / reduction per step, no saved full parameter, backward
re-materialisation, prefetch boundaries at `v_proj` and `down_proj`) are exercised by a model
small enough for exhaustive tests (reference: `src/sharded_runtime/runtime/engine.py:352-490`,
`src/sharded_runtime/runtime/operators.py:11-103`).
"""

from __future__ import annotations

import types

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

from shardtrain_b200.models.transformer_block import causal_attention_heads, gated_mlp
from shardtrain_b200.parallel.model import ROW_PROJECTIONS, supported_blocks, validate_blocks
from shardtrain_b200.runtime.engine import UnitState
from shardtrain_b200.runtime.qwen2_adapter import ParameterPartition
from shardtrain_b200.runtime.qwen2_operators import Branch, ColumnProjection, NormFn, RowLinear

BLOCK_PARAMETERS = (
    ("attention_norm.weight", None), ("attention.q_proj.weight", 0), ("attention.k_proj.weight", 0),
    ("attention.v_proj.weight", 0), ("attention.out_proj.weight", 1), ("mlp_norm.weight", None),
    ("mlp.up_proj.weight", 0), ("mlp.gate_proj.weight", 0), ("mlp.down_proj.weight", 1),
)


def _column(runtime, unit, prefix, names, x, role):
    branches = [Branch(unit.handle(prefix + n + ".weight")) for n in names]
    weights = [unit.forward_weight(b.weight.spec.param_id) for b in branches]
    with runtime.tp.tagged(role):
        return ColumnProjection.apply(x, runtime, tuple(branches), branches[-1].weight, *weights)


def _row(runtime, unit, name, x):
    handle = unit.handle(name)
    return RowLinear.apply(x, unit.forward_weight(name), runtime, handle, False)


def _norm(unit, name, x, eps):
    handle = unit.handle(name)
    return NormFn.apply(x, unit.forward_weight(name), handle, eps)


def block_forward(runtime, unit, block, prefix, x):
    """Pre-norm attention + SwiGLU block on materialised TP-local weights."""
    if x.ndim != 3 or x.shape[-1] != block.hidden_size:
        raise ValueError(f"Expected [batch, sequence, {block.hidden_size}], got {tuple(x.shape)}")
    unit.pre_forward()
    attention = block.attention
    h = _norm(unit, prefix + "attention_norm.weight", x, block.attention_norm.eps)
    q, k, v = _column(runtime, unit, prefix + "attention.", ("q_proj", "k_proj", "v_proj"), h, "qkv")
    mixed = causal_attention_heads(q, k, v, attention.head_dim)
    x = x + _row(runtime, unit, prefix + "attention.out_proj.weight", mixed)
    h = _norm(unit, prefix + "mlp_norm.weight", x, block.mlp_norm.eps)
    gate, up = _column(runtime, unit, prefix + "mlp.", ("gate_proj", "up_proj"), h, "gate_up")
    x = x + _row(runtime, unit, prefix + "mlp.down_proj.weight", gated_mlp(gate, up))
    return unit.post_forward(x)


@torch.no_grad()
def register_blocks(runtime, model, mesh=None, *, sp=False):
    if getattr(model, "_tp_plan", None) is not None:
        raise ValueError("Register the original dense model, before TP or optimizer construction")
    blocks = supported_blocks(model)
    runtime.bind_groups(mesh, sp)
    tp, fsdp = runtime.tp, runtime.materializer
    if tp.degree not in {1, 2, 4}:
        raise ValueError("TP supports degree 1, 2 or 4")
    if sp and tp.degree == 1:
        raise ValueError("SP requires TP degree > 1")
    parameters = validate_blocks(model, blocks, tp.degree)
    model.to(runtime.device)
    runtime.model = model
    runtime.compute_dtype = torch.float32
    runtime.comm.phase = "INIT"
    # one canonical dense source: rank 0's values reach every rank before slicing
    if dist.is_initialized():
        for _, parameter in parameters:
            runtime.comm.issue(
                "world", "init_broadcast", dist.group.WORLD, parameter, parameter,
                lambda async_, p=parameter: dist.broadcast(p, src=0, async_op=async_),
                channel="fsdp_ag", asynchronous=False,
            )
    sequential = type(model) is nn.Sequential
    owners, values, runtime.partitions = {}, {}, {}
    for index, block in enumerate(blocks):
        unit = UnitState(runtime, index, block)
        runtime.units.append(unit)
        prefix = f"{index}." if sequential else ""
        for local_name, dim in BLOCK_PARAMETERS:
            module_path, attr = local_name.rsplit(".", 1)
            module = block.get_submodule(module_path)
            parameter = getattr(module, attr)
            part = ParameterPartition(tuple(parameter.shape), dim, tp.rank, tp.degree)
            name = prefix + local_name
            runtime.partitions[name] = part
            local = part.local_slice(parameter.detach()).contiguous()
            layout = {0: "column", 1: "row", None: "replicated"}[dim]
            runtime.add_parameter(unit, name, local, tuple(parameter.shape), layout)
            owners[name], values[name] = (module, attr), local
        unit.forward_prefetch_handle = runtime.registry[prefix + "attention.v_proj.weight"]
        unit.backward_prefetch_handle = runtime.registry[prefix + "mlp.down_proj.weight"]
    runtime.allocate_arenas()
    for name, handle in runtime.registry.items():
        q, keep = handle.spec.fsdp_shard_numel, handle.spec.valid_len(fsdp.rank)
        if keep:
            handle.local_shard.data[:keep].copy_(values[name].reshape(-1)[fsdp.rank * q: fsdp.rank * q + keep])
        module, attr = owners[name]
        module._parameters[attr] = handle.local_shard
        handle.pending_value = None
    for index, block in enumerate(blocks):
        block.attention.num_heads //= tp.degree
        prefix = f"{index}." if sequential else ""
        unit = runtime.units[index]
        block.forward = types.MethodType(
            lambda self, x, _u=unit, _p=prefix: block_forward(runtime, _u, self, _p, x), block)
    model._sharded_runtime = runtime
    return runtime
