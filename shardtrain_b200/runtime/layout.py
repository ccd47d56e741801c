"""Shard layout: per-parameter flat FP32 shards, the rank-major packed gather buffer, the
destination-major packed gradient buffer, and the flat arenas that back every shard leaf.

Contract (identical to the reference, `src/sharded_runtime/runtime/layout.py:9-106` and
`docs/fsdp_copy_out_layout.md`): a TP-local tensor of n elements is flattened and cut into F
shards of q = ceil(n / F) elements; rank r owns [r*q, (r+1)*q), zero padded past n.  The packed
all-gather buffer is rank-major (rank r's slot holds its shards of all the unit's parameters back
to back); the packed reduce-scatter input is destination-major with the same slot layout.

What is new here: every shard leaf is a view into one flat arena per runtime (parameters and
gradients), so a single kernel launch can sweep all leaves (optimizer, finite check) and the
sm_100a gather / reduce-scatter kernels address shards by (arena base, offset) through a
`segment_table`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch
from torch import Tensor, nn

ALIGN = 8  # elements; keeps fp32 shards 32-byte and their bf16 shadows 16-byte aligned


@dataclass(frozen=True)
class ParameterSpec:
    param_id: str
    unit_id: int
    global_shape: tuple[int, ...]
    tp_local_shape: tuple[int, ...]
    tp_layout: str            # "column" | "row" | "replicated"
    tp_grad_reduce: str       # "sum" for TP-replicated parameters, else "none"
    numel: int
    fsdp_shard_numel: int
    padding_numel: int
    dtype: torch.dtype

    @classmethod
    def create(cls, name, unit_id, weight, global_shape, layout, degree) -> "ParameterSpec":
        n = weight.numel()
        q = -(-n // degree)
        return cls(name, unit_id, tuple(global_shape), tuple(weight.shape), layout,
                   "sum" if layout == "replicated" else "none", n, q, degree * q - n, weight.dtype)

    def valid_len(self, rank: int) -> int:
        return max(0, min(self.fsdp_shard_numel, self.numel - rank * self.fsdp_shard_numel))


@dataclass
class ShardedParameter:
    """Handle of one parameter: spec, the persistent shard leaf and its arena placement."""

    spec: ParameterSpec
    local_shard: nn.Parameter
    unit: object = None
    grad_ready_event: object = None
    grad_step: int = -1
    forward_uses: int = 0
    arena_offset: int = 0            # element offset of the shard in the runtime arenas
    grad_shard: Tensor | None = None  # persistent gradient view (same offset, gradient arena)

    def weight(self):
        """Current-generation full parameter; only legal while the unit is in backward."""
        return self.unit.weight(self.spec.param_id)

    def mark_forward(self, *, tied_second_use: bool = False) -> None:
        if tied_second_use:
            if self.forward_uses != 1 or self.unit.state != "FWD_ACTIVE":
                raise RuntimeError("Tied LM head must consume the embedding owner exactly once")
        elif self.forward_uses or self.unit.state != "FWD_ACTIVE":
            raise RuntimeError(f"Repeated/early parameter consumer {self.spec.param_id}")
        self.forward_uses += 1


def shard_of(weight: Tensor, spec: ParameterSpec, rank: int, out: Tensor | None = None) -> Tensor:
    """Rank `rank`'s zero-padded shard of a TP-local tensor (written into `out` when given)."""
    q = spec.fsdp_shard_numel
    shard = torch.zeros(q, dtype=weight.dtype, device=weight.device) if out is None else out.zero_()
    keep = spec.valid_len(rank)
    if keep:
        shard[:keep].copy_(weight.detach().reshape(-1)[rank * q : rank * q + keep])
    return shard


def initialize_shard(weight: Tensor, spec: ParameterSpec, rank: int) -> nn.Parameter:
    return nn.Parameter(shard_of(weight, spec, rank))


def offsets(specs: Sequence[ParameterSpec]) -> tuple[list[int], int]:
    """Start of each parameter's shard inside one rank's slot, and the slot length."""
    starts, cursor = [], 0
    for spec in specs:
        starts.append(cursor)
        cursor += spec.fsdp_shard_numel
    return starts, cursor


_PACK_TABLES: dict[tuple, tuple[Tensor, list[int]]] = {}


def _native_packing(buffer: Tensor, specs: Sequence[ParameterSpec]) -> bool:
    """The single-launch pack / unpack kernels serve fp32 buffers on a GPU with the extension
    built; everything else (CPU, other dtypes) takes the torch path below."""
    if not buffer.is_cuda or buffer.dtype != torch.float32 or not specs:
        return False
    from shardtrain_b200 import ops

    return ops.extension_path() is not None and all(s.dtype == torch.float32 for s in specs)


def _pack_table(specs: Sequence[ParameterSpec], device) -> tuple[Tensor, list[int]]:
    """Device table {start in slot, q, numel, offset in the flat output} per parameter, plus the
    output offsets on the host; built once per unit and device."""
    key = (tuple((s.param_id, s.numel, s.fsdp_shard_numel) for s in specs), str(device))
    hit = _PACK_TABLES.get(key)
    if hit is None:
        starts, _ = offsets(specs)
        rows, cursor, outs = [], 0, []
        for spec, start in zip(specs, starts):
            rows.append([start, spec.fsdp_shard_numel, spec.numel, cursor])
            outs.append(cursor)
            cursor += _round_up(spec.numel, ALIGN)
        outs.append(cursor)
        hit = (torch.tensor(rows, dtype=torch.int64, device=device), outs)
        _PACK_TABLES[key] = hit
    return hit


def copy_out(storage: Tensor, specs: Sequence[ParameterSpec], degree: int) -> dict[str, Tensor]:
    """Rank-major packed gather buffer -> one independent tensor per parameter, padding dropped.
    On a GPU one kernel launch writes all the unit's parameters into one flat buffer (the
    returned tensors are views of it); elsewhere one copy per parameter."""
    starts, slot = offsets(specs)
    if storage.numel() != degree * slot:
        raise RuntimeError("Packed gather buffer has the wrong length")
    if _native_packing(storage, specs):
        from shardtrain_b200 import ops

        table, outs = _pack_table(specs, storage.device)
        flat = torch.empty(outs[-1], dtype=storage.dtype, device=storage.device)
        ops.load().unpack_gathered(storage.reshape(-1), slot, table, max(s.numel for s in specs), flat)
        return {spec.param_id: flat[off : off + spec.numel].view(spec.tp_local_shape)
                for spec, off in zip(specs, outs)}
    by_rank = storage.view(degree, slot)
    result = {}
    for spec, start in zip(specs, starts):
        q = spec.fsdp_shard_numel
        # [degree, q] -> flat [degree*q]; the first numel elements are the parameter
        full = by_rank[:, start : start + q].reshape(-1)[: spec.numel].clone()
        result[spec.param_id] = full.view(spec.tp_local_shape)
    return result


def pack_gradients(grads: Sequence[Tensor], specs: Sequence[ParameterSpec], degree: int) -> Tensor:
    """Full per-parameter gradients -> destination-major, zero padded reduce-scatter input."""
    starts, slot = offsets(specs)
    for grad, spec in zip(grads, specs):
        if tuple(grad.shape) != spec.tp_local_shape or grad.dtype != spec.dtype:
            raise RuntimeError(f"Invalid full gradient: {spec.param_id}")
    if _native_packing(grads[0], specs):
        from shardtrain_b200 import ops

        table, _ = _pack_table(specs, grads[0].device)
        held = [g.contiguous() for g in grads]                  # alive until the launch is queued
        pointers = torch.tensor([g.data_ptr() for g in held], dtype=torch.int64).to(grads[0].device)
        packed = torch.empty(degree * slot, dtype=torch.float32, device=grads[0].device)
        ops.load().pack_gradients(pointers, table, degree, slot, slot,
                                  max(s.fsdp_shard_numel for s in specs), packed)
        for g in held:
            g.record_stream(torch.cuda.current_stream(g.device))
        return packed
    packed = grads[0].new_zeros(degree, slot)
    for grad, spec, start in zip(grads, specs, starts):
        q = spec.fsdp_shard_numel
        flat = grad.reshape(-1)
        whole = spec.numel // q
        if whole:
            packed[:whole, start : start + q].copy_(flat[: whole * q].view(whole, q))
        tail = spec.numel - whole * q
        if tail:
            packed[whole, start : start + tail].copy_(flat[whole * q :])
    return packed.view(-1)


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@dataclass
class ArenaPlan:
    """Placement of every shard inside the flat arenas, unit-major."""

    offsets: dict[str, int] = field(default_factory=dict)
    unit_ranges: dict[int, tuple[int, int]] = field(default_factory=dict)
    total: int = 0

    def add(self, spec: ParameterSpec) -> int:
        start = _round_up(self.total, ALIGN)
        self.offsets[spec.param_id] = start
        self.total = start + spec.fsdp_shard_numel
        lo, _ = self.unit_ranges.get(spec.unit_id, (start, start))
        self.unit_ranges[spec.unit_id] = (lo, self.total)
        return start

    def padded_total(self) -> int:
        return _round_up(max(self.total, ALIGN), ALIGN)


def padding_ranges(handles: Sequence[ShardedParameter], rank: int) -> list[tuple[int, int]]:
    """Arena ranges that must hold exact zeros: each shard's tail past its valid length."""
    out = []
    for h in handles:
        keep = h.spec.valid_len(rank)
        if keep < h.spec.fsdp_shard_numel:
            out.append((h.arena_offset + keep, h.arena_offset + h.spec.fsdp_shard_numel))
    return out


def segment_table(handles: Sequence[ShardedParameter], full_offsets: dict[str, int],
                  keep_fp32: set[str], *, mark_replicated: bool = False) -> Tensor:
    """CPU int64 [n, 5] rows (shard_off, q, numel, full_off, flags) for the gather and
    reduce-scatter kernels; offsets are in elements from the arena / full-buffer base.  Flag bit 0:
    keep FP32 when materialising; bit 1 (reduce tables, `mark_replicated`): the parameter is
    replicated over the TP axis, so its gradient is summed over the whole mesh."""
    rows = [
        [h.arena_offset, h.spec.fsdp_shard_numel, h.spec.numel, full_offsets[h.spec.param_id],
         (1 if h.spec.param_id in keep_fp32 else 0)
         | (2 if mark_replicated and h.spec.tp_grad_reduce == "sum" else 0)]
        for h in handles
    ]
    return torch.tensor(rows, dtype=torch.int64).reshape(len(rows), 5)
