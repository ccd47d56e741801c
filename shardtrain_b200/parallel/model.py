"""Legacy synchronous TP/SP conversion of the toy block model.

`parallelize_tp_sp` accepts only the original `TransformerBlock` (or an `nn.Sequential` of them):
it broadcasts every dense parameter from TP rank 0, swaps the seven projections for
column / row parallel linears, divides the head count, and (with SP) installs one shared gather
per projection group.  `TensorParallelPlan` carries the per-parameter partitions and the loss /
gradient conventions of that path (`src/sharded_runtime/parallel/model.py:24-158`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor, nn

from shardtrain_b200.models.transformer_block import CausalSelfAttention, RMSNorm, SwiGLU, TransformerBlock
from shardtrain_b200.parallel.mappings import TPGroup
from shardtrain_b200.parallel.shared_projection import SharedProjectionGroup
from shardtrain_b200.parallel.tp_linear import ColumnParallelLinear, ParameterPartition, RowParallelLinear

ROW_PROJECTIONS = {"out_proj", "down_proj"}
BLOCK_CHILDREN = {"attention_norm": RMSNorm, "attention": CausalSelfAttention,
                  "mlp_norm": RMSNorm, "mlp": SwiGLU}
PROJECTIONS = {"attention": {"q_proj", "k_proj", "v_proj", "out_proj"},
               "mlp": {"gate_proj", "up_proj", "down_proj"}}


@dataclass(frozen=True)
class TensorParallelPlan:
    model: nn.Module
    group: TPGroup
    sp: bool
    partitions: dict[str, ParameterPartition]

    def input_for_rank(self, full_batch: Tensor) -> Tensor:
        return self.group.sequence_shard(full_batch) if self.sp else full_batch

    def backward_loss(self, output: Tensor) -> Tensor:
        return output.square().mean() / (self.group.degree if self.sp else 1)

    def reported_loss(self, local_loss: Tensor) -> Tensor:
        return self.group.sum(local_loss.detach()) if self.sp else local_loss.detach()

    def finalize_gradients(self) -> None:
        """Once per optimizer step, after all micro-batch backwards: under SP every rank saw only
        its tokens, so replicated parameters need the SUM of their gradients."""
        if not self.sp:
            return
        for name, parameter in self.model.named_parameters():
            if self.partitions[name].dim is None:
                if parameter.grad is None:
                    raise RuntimeError(f"Replicated parameter gradient is missing: {name}")
                parameter.grad = self.group.sum(parameter.grad)

    def global_parameters(self, *, gradients: bool = False) -> dict[str, Tensor]:
        """Reassemble canonical tensors (tests only)."""
        out = {}
        for name, parameter in self.model.named_parameters():
            tensor = parameter.grad if gradients else parameter
            if tensor is None:
                raise RuntimeError(f"No gradient available for {name}")
            dim = self.partitions[name].dim
            out[name] = tensor.detach().clone() if dim is None else self.group.gather(tensor.detach(), dim=dim)
        return out


def supported_blocks(model: nn.Module) -> list[TransformerBlock]:
    if type(model) is TransformerBlock:
        return [model]
    if type(model) is nn.Sequential and len(model) and all(type(b) is TransformerBlock for b in model):
        return list(model)
    raise ValueError("M1 only supports TransformerBlock or Sequential of original Blocks")


def validate_blocks(model: nn.Module, blocks, degree: int) -> list[tuple[str, nn.Parameter]]:
    parameters = list(model.named_parameters(remove_duplicate=False))
    if len({id(p) for _, p in parameters}) != len(parameters):
        raise ValueError("Shared parameters are not supported by M1 conversion")
    if len(parameters) != 9 * len(blocks):
        raise ValueError("M1 requires exactly the original nine parameters per Block")
    if any(p.dtype != torch.float32 or not p.requires_grad or p.grad is not None for _, p in parameters):
        raise ValueError("M1 conversion requires untrained, trainable FP32 parameters")
    for block in blocks:
        children = dict(block.named_children())
        if set(children) != set(BLOCK_CHILDREN) or any(
                type(children[n]) is not cls for n, cls in BLOCK_CHILDREN.items()):
            raise ValueError("M1 requires original Block submodules without custom replacements")
        if block.attention.num_heads % degree:
            raise ValueError("Attention heads must be divisible by TP degree")
        for owner, names in PROJECTIONS.items():
            module = getattr(block, owner)
            if set(dict(module.named_children())) != names:
                raise ValueError("M1 requires the original attention/MLP projection set")
            for name, linear in module.named_children():
                if type(linear) is not nn.Linear or linear.bias is not None:
                    raise ValueError("Only original bias-free Block projections are supported")
                if linear.weight.shape[1 if name in ROW_PROJECTIONS else 0] % degree:
                    raise ValueError("Projection partition dimension is not divisible by TP degree")
    return parameters


def parallelize_tp_sp(model: nn.Module, tp_group: Any = None, *, sp: bool = False,
                      broadcast_fn=None) -> TensorParallelPlan:
    """Convert `model` in place (before its optimizer exists) and return the plan."""
    if hasattr(model, "_tp_plan"):
        raise ValueError("Module is already TP-parallelized")
    blocks = supported_blocks(model)
    group = TPGroup.from_process_group(tp_group)
    if group.degree not in {1, 2, 4}:
        raise ValueError("TP supports degree 1, 2 or 4")
    if sp and group.degree == 1:
        raise ValueError("SP requires TP degree > 1")
    parameters = validate_blocks(model, blocks, group.degree)
    with torch.no_grad():
        for _, parameter in parameters:
            if broadcast_fn is None:
                group.broadcast(parameter)
            else:
                broadcast_fn(parameter, group)
    for block in blocks:
        for owner in PROJECTIONS:
            module = getattr(block, owner)
            for name, linear in list(module.named_children()):
                cls = RowParallelLinear if name in ROW_PROJECTIONS else ColumnParallelLinear
                setattr(module, name, cls(linear, group, sp=sp))
        block.attention.num_heads //= group.degree
        if sp:
            a, m = block.attention, block.mlp
            a.projection_group = SharedProjectionGroup((a.q_proj, a.k_proj, a.v_proj), group, "qkv")
            m.projection_group = SharedProjectionGroup((m.gate_proj, m.up_proj), group, "gate_up")
    partitions = {}
    for name, parameter in model.named_parameters():
        owner = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        partitions[name] = (owner.partition if isinstance(owner, (ColumnParallelLinear, RowParallelLinear))
                            else ParameterPartition(tuple(parameter.shape), None, group.rank, group.degree))
    plan = TensorParallelPlan(model, group, sp, partitions)
    model._tp_plan = plan
    return plan
