"""Save / resume for the sharded runtime (the reference has a loader only).

Two formats, both safetensors written by `models.qwen2_checkpoint.save_safetensors`:

* sharded -- one file per rank holding that rank's flat FP32 shard of every parameter under its
  Hugging Face name, plus `exp_avg.` / `exp_avg_sq.` copies when an arena AdamW is bound, and a
  JSON sidecar with the mesh, every `ParameterSpec`, and step counters.  Loading on the same
  mesh is bit-exact and needs no communication.
* full -- canonical HF tensors: the F shards of each TP-local tensor are concatenated (valid
  prefixes only) and the T pieces are concatenated along the partition dimension
  (`src/sharded_runtime/runtime/engine.py:696-709`,
  `experiments/fsdp4_hybrid_2x2/worker.py:157-179`).  Rank 0 writes `model.safetensors`, which
  the strict reader accepts, so a run can resume on a different F x T mesh; optimizer moments
  are exported the same way (`optimizer.safetensors`) and re-sharded on load.
"""

from __future__ import annotations

import json
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200.models.qwen2_checkpoint import SafetensorsFile, save_safetensors


def _moments(optimizer):
    if optimizer is None or not hasattr(optimizer, "exp_avg"):
        return {}
    return {"exp_avg": optimizer.exp_avg, "exp_avg_sq": optimizer.exp_avg_sq}


def sharded_state_dict(runtime, optimizer=None) -> dict[str, torch.Tensor]:
    """HF name -> this rank's flat FP32 shard (optimizer moments under `exp_avg.` prefixes)."""
    state = {name: h.local_shard.detach() for name, h in runtime.registry.items()}
    for tag, arena in _moments(optimizer).items():
        for name, h in runtime.registry.items():
            state[f"{tag}.{name}"] = arena.narrow(0, h.arena_offset, h.spec.fsdp_shard_numel)
    return state


def _coordinates(runtime):
    return runtime.materializer.rank, runtime.tp.rank


def _refuse_failed(runtime):
    """A FAILED runtime may hold a half-applied or non-finite update (the fused AdamW runs inside
    the last reduction, before the step's finite vote is read): its state must never be saved."""
    if runtime.failed:
        raise RuntimeError("Refusing to save a checkpoint from a FAILED runtime: its shards may "
                           "hold the update of the step that failed")


def save_sharded(runtime, directory, optimizer=None, *, trainer_step=None, trainer=None) -> Path:
    """`trainer` (optional): its step counter and loss-scaler state are stored too and restored
    by `load_sharded(..., trainer=...)`."""
    _refuse_failed(runtime)
    if trainer is not None and trainer_step is None:
        trainer_step = trainer.step_id
    scaler = getattr(trainer, "scaler", None)
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    f, t = _coordinates(runtime)
    tag = f"f{f}t{t}"
    state = {k: v.cpu().clone() for k, v in sharded_state_dict(runtime, optimizer).items()}
    save_safetensors(directory / f"shard.{tag}.safetensors", state)
    meta = {
        "fsdp_degree": runtime.materializer.degree, "tp_degree": runtime.tp.degree,
        "fsdp_rank": f, "tp_rank": t, "runtime_step": runtime.step_id,
        "parameter_version": runtime.parameter_shards_version,
        "optimizer_step": getattr(optimizer, "arena_step", None), "trainer_step": trainer_step,
        "scaler": scaler.state_dict() if scaler is not None and scaler.is_enabled() else None,
        "specs": {n: {**{k: (str(v) if k == "dtype" else v) for k, v in asdict(h.spec).items()}}
                  for n, h in runtime.registry.items()},
    }
    (directory / f"meta.{tag}.json").write_text(json.dumps(meta, indent=1))
    return directory


@torch.no_grad()
def load_sharded(runtime, directory, optimizer=None, *, trainer=None) -> dict:
    """Restore this rank's shards (and moments) written on the same F x T mesh, between steps.

    Also restored: the optimizer's step count, the runtime's step counter (so event logs and
    leases continue the saved numbering) and, with `trainer`, its step counter and loss-scaler
    state.  On sm_100a the bf16 shadow of the shards is marked stale, so the next gather first
    rebuilds it from the loaded FP32 masters."""
    if runtime.active:
        raise RuntimeError("load_sharded must run between steps")
    directory = Path(directory)
    f, t = _coordinates(runtime)
    tag = f"f{f}t{t}"
    meta = json.loads((directory / f"meta.{tag}.json").read_text())
    if (meta["fsdp_degree"], meta["tp_degree"]) != (runtime.materializer.degree, runtime.tp.degree):
        raise ValueError("Sharded checkpoint was written on a different mesh; load the full format")
    reader = SafetensorsFile(directory / f"shard.{tag}.safetensors")
    for name, h in runtime.registry.items():
        spec = meta["specs"].get(name)
        if spec is None or spec["fsdp_shard_numel"] != h.spec.fsdp_shard_numel:
            raise ValueError(f"Checkpoint shard does not match the registered layout: {name}")
        h.local_shard.data.copy_(reader.tensor(name))
    for tag_name, arena in _moments(optimizer).items():
        for name, h in runtime.registry.items():
            arena.narrow(0, h.arena_offset, h.spec.fsdp_shard_numel).copy_(reader.tensor(f"{tag_name}.{name}"))
    if optimizer is not None and meta.get("optimizer_step") is not None:
        optimizer.arena_step = meta["optimizer_step"]
        for state in getattr(optimizer, "state", {}).values():
            if "step" in state:
                state["step"].fill_(float(meta["optimizer_step"]))
    if meta.get("runtime_step") is not None:
        runtime.step_id = runtime.comm.step_id = int(meta["runtime_step"])
    if trainer is not None:
        if meta.get("trainer_step") is not None:
            trainer.step_id = int(meta["trainer_step"])
        if meta.get("scaler") and trainer.scaler.is_enabled():
            trainer.scaler.load_state_dict(meta["scaler"])
    runtime.parameter_shards_version += 1
    runtime.publish_parameter_shards_ready("checkpoint_load")
    return meta


def _gather_tp(runtime, name, local):
    part = runtime.qwen_partitions[name] if hasattr(runtime, "qwen_partitions") else runtime.partitions[name]
    tp = runtime.tp
    if part.dim is None or tp.degree == 1:
        return local
    pieces = runtime.verification_gather(local.contiguous(), tp.process_group, "tp")
    return torch.cat(pieces, dim=part.dim)


def full_state_dict(runtime, optimizer=None) -> dict[str, torch.Tensor]:
    """Canonical tensors on every rank (collective: all ranks must call it)."""
    out = {}
    sources = {"": None, **_moments(optimizer)}
    for prefix, arena in sources.items():
        for name, h in runtime.registry.items():
            shard = h.local_shard.detach() if arena is None else arena.narrow(
                0, h.arena_offset, h.spec.fsdp_shard_numel)
            parts = runtime.verification_gather(shard.contiguous(), runtime.materializer.group, "fsdp")
            flat = torch.cat([p[: h.spec.valid_len(r)] for r, p in enumerate(parts)])
            key = name if not prefix else f"{prefix}.{name}"
            out[key] = _gather_tp(runtime, name, flat.view(h.spec.tp_local_shape))
    return out


def save_full(runtime, directory, optimizer=None) -> Path:
    """Rank 0 writes `model.safetensors` (+ `optimizer.safetensors`); every rank participates."""
    _refuse_failed(runtime)
    directory = Path(directory)
    state = full_state_dict(runtime, optimizer)
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        directory.mkdir(parents=True, exist_ok=True)
        weights = {k: v.cpu() for k, v in state.items() if not k.startswith("exp_avg")}
        save_safetensors(directory / "model.safetensors", weights, {"format": "pt"})
        moments = {k: v.cpu() for k, v in state.items() if k.startswith("exp_avg")}
        if moments:
            save_safetensors(directory / "optimizer.safetensors", moments,
                             {"optimizer_step": str(getattr(optimizer, "arena_step", 0))})
    if dist.is_initialized():
        dist.barrier()
    return directory


@torch.no_grad()
def load_full_optimizer(runtime, directory, optimizer) -> None:
    """Re-shard canonical AdamW moments onto the current mesh."""
    reader = SafetensorsFile(Path(directory) / "optimizer.safetensors")
    fsdp_rank = runtime.materializer.rank
    parts = getattr(runtime, "qwen_partitions", None) or runtime.partitions
    for tag, arena in _moments(optimizer).items():
        for name, h in runtime.registry.items():
            local = parts[name].local_slice(reader.tensor(f"{tag}.{name}")).contiguous().reshape(-1)
            q, keep = h.spec.fsdp_shard_numel, h.spec.valid_len(fsdp_rank)
            view = arena.narrow(0, h.arena_offset, q)
            view.zero_()
            if keep:
                view[:keep].copy_(local[fsdp_rank * q: fsdp_rank * q + keep])
    optimizer.arena_step = int(reader.metadata.get("optimizer_step", 0))
