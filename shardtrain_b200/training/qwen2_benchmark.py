"""Qwen2 training benchmark: train the configured model and leave one JSON record per rank.

Command line and artifacts follow the reference benchmark
(`src/sharded_runtime/training/qwen2_benchmark.py:173-492`): `--config`, `--warmup`,
`--profile-mode off|torch|nsight`, `--profile-detail`, `--runtime-events auto|on|off`,
`--peak-tflops-per-gpu` and `--section.field value` overrides; outputs
`benchmark.rank{r}.json` (per-step rows, p50/p95, tokens/s, memory, ownership audit, FLOP
summary), `gpu_topology.txt` on rank 0, plus whatever the profile capture writes.  An output
directory that already holds records of this rank is refused.

Every step is timed three ways: host wall clock including the end-of-step device synchronise,
the maximum of that over ranks (reduced outside the timed interval), and a CUDA-event span.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.metadata
import json
import math
import platform
import subprocess
import time
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200.config import Config, ConfigError, load_config
from shardtrain_b200.distributed.context import WorkerEnvironment
from shardtrain_b200.launch.bootstrap import WorkerSession
from shardtrain_b200.models.qwen2_factory import build_qwen_model
from shardtrain_b200.observability.metadata import write_json
from shardtrain_b200.observability.profiling import ProfileCapture
from shardtrain_b200.runtime.engine import ShardedRuntime
from shardtrain_b200.training.performance import qwen_performance_summary
from shardtrain_b200.training.qwen2_precision import resolve_qwen_compute_dtype
from shardtrain_b200.training.qwen2_trainer import QwenTrainer

RECORD_PREFIXES = ("environment", "benchmark", "profiling")


def percentile(values, quantile):
    """Linear-interpolated quantile of a small sample; None for an empty one."""
    if not values:
        return None
    ordered = sorted(values)
    where = (len(ordered) - 1) * quantile
    below = int(math.floor(where))
    above = min(below + 1, len(ordered) - 1)
    return ordered[below] + (ordered[above] - ordered[below]) * (where - below)


def _package_version(name):
    try:
        return importlib.metadata.version(name)
    except importlib.metadata.PackageNotFoundError:
        return None


def software_versions() -> dict:
    nccl = None
    if dist.is_nccl_available() and torch.cuda.is_available():
        nccl = torch.cuda.nccl.version()
    return {
        "torch": torch.__version__,
        "cuda_build": torch.version.cuda,
        "nccl": nccl,
        "packages": {name: _package_version(name) for name in ("transformers", "safetensors")},
        "platform": platform.platform(),
    }


def describe_model_source(config: Config, model) -> dict:
    tied = model.lm_head.weight is model.model.embed_tokens.weight
    checkpoint = config.model.checkpoint_path
    info = {
        "initialization": "local_safetensors" if checkpoint else "random",
        "checkpoint_path": str(Path(checkpoint).resolve()) if checkpoint else None,
        "seed": config.training.seed,
        "memory_strategy": "meta construction; one host source parameter at a time, copied "
                           "straight into the persistent FP32 TP/FSDP shard arena",
        "tied_aliases": {"lm_head.weight": "model.embed_tokens.weight"} if tied else {},
        "config": model.config.to_dict(),
        "global_unique_parameter_numel": sum(p.numel() for p in model.parameters()),
        "actual_checkpoint_logits_reference_verified": False,
    }
    if config.model.hf_config_path:
        path = Path(config.model.hf_config_path).resolve()
        info["hf_config_path"] = str(path)
        info["hf_config_sha256"] = hashlib.sha256(path.read_bytes()).hexdigest()
        provenance = path.with_suffix(".provenance.json")
        if provenance.is_file():
            info["config_provenance"] = json.loads(provenance.read_text(encoding="utf-8"))
    return info


def record_gpu_topology(session) -> None:
    """Rank 0 on CUDA stores the NVLink / PCIe matrix printed by `nvidia-smi topo -m`."""
    if session.worker.rank != 0 or session.context.device.type != "cuda":
        return
    command = ["nvidia-smi", "topo", "-m"]
    status = {"command": " ".join(command)}
    try:
        done = subprocess.run(command, capture_output=True, text=True, check=False, timeout=15)
        text, status["returncode"] = done.stdout + done.stderr, done.returncode
    except (OSError, subprocess.TimeoutExpired) as exc:
        text, status["error"] = str(exc), repr(exc)
    (session.directory / "gpu_topology.txt").write_text(text, encoding="utf-8")
    write_json(session.directory / "gpu_topology_status.json", status)


def max_over_ranks(runtime, seconds: float, world_size: int) -> float:
    """Slowest rank's step time; goes through the coordinator so it is ordered like any other
    collective of its process group."""
    if world_size == 1:
        return seconds
    value = torch.tensor(seconds, dtype=torch.float64, device=runtime.device)
    comm = runtime.comm
    comm.unit_id, comm.phase = None, "BENCHMARK"
    comm.issue(
        "world", "benchmark_max_rank_seconds", dist.group.WORLD, value, value,
        lambda async_op: dist.all_reduce(value, op=dist.ReduceOp.MAX, group=dist.group.WORLD,
                                         async_op=async_op),
        channel="fsdp_rs", asynchronous=False, group_role="benchmark_metadata",
    )
    return float(value.item())


def memory_counters(device: torch.device) -> dict:
    if device.type != "cuda":
        return dict.fromkeys(("max_allocated", "max_reserved", "allocated_end", "reserved_end"))
    return {
        "max_allocated": torch.cuda.max_memory_allocated(device),
        "max_reserved": torch.cuda.max_memory_reserved(device),
        "allocated_end": torch.cuda.memory_allocated(device),
        "reserved_end": torch.cuda.memory_reserved(device),
    }


def ownership_audit(runtime, trainer) -> dict:
    """What this rank owns persistently, and whether the runtime's invariants held."""
    leaves = runtime.sharded_parameters()
    rank = runtime.materializer.rank
    state_bytes = sum(t.numel() * t.element_size()
                      for per_leaf in trainer.optimizer.state.values()
                      for t in per_leaf.values()
                      if isinstance(t, torch.Tensor) and t.numel() > 1)
    return {
        "unit_count": len(runtime.units),
        "persistent_shard_count": len(leaves),
        "persistent_shard_numel_including_padding": sum(p.numel() for p in leaves),
        "persistent_shard_valid_numel": sum(h.spec.valid_len(rank) for h in runtime.registry.values()),
        "parameter_bytes": sum(p.numel() * p.element_size() for p in leaves),
        "gradient_bytes": sum(p.grad.numel() * p.grad.element_size() for p in leaves
                              if p.grad is not None),
        "optimizer_tensor_bytes": state_bytes,
        "optimizer_state_parameter_count": len(trainer.optimizer.state),
        "parameter_dtypes": sorted({str(p.dtype) for p in leaves}),
        "master_weight_strategy": "persistent FP32 shard arena is the optimizer's master copy",
        "executor": runtime.executor.name,
        "live_buffers": len(runtime.comm.live_buffers),
        "live_fullparam_leases": sum(u.lease is not None for u in runtime.units),
        "units_reduced_once_last_microbatch": all(u.reductions == 1 for u in runtime.units),
        "stable_shard_identity": all(
            (id(h.local_shard), h.local_shard.data_ptr()) == runtime.identities[name]
            for name, h in runtime.registry.items()),
    }


PRECISION_POLICY_ROLES = {
    "parameters": "fp32", "parameter_all_gather": "fp32", "gradient_reduce": "fp32",
    "optimizer_state": "fp32", "norm_accumulation": "fp32", "loss": "fp32",
    "sp_backward_input_grad_reduce_scatter": "fp32",
}
COMPUTE_DTYPE_ROLES = ("compute", "linear_backward", "sp_forward_input_all_gather",
                       "sp_forward_output_reduce_scatter", "sp_backward_output_grad_all_gather")


def _check_arguments(config, warmup, profile_mode, profile_detail, peak):
    if config.model.model_type != "qwen2":
        raise ConfigError("Qwen benchmark requires model.model_type=qwen2")
    if type(warmup) is not int or warmup < 0:
        raise ConfigError("warmup must be a nonnegative integer")
    if profile_mode not in {"off", "torch", "nsight"}:
        raise ConfigError("profile_mode must be off, torch, or nsight")
    if profile_detail not in {"low_overhead", "full"}:
        raise ConfigError("profile_detail must be low_overhead or full")
    if profile_mode == "nsight" and config.parallel.device != "cuda":
        raise ConfigError("Nsight capture requires CUDA; use torch or off for CPU")
    if peak is not None and (not math.isfinite(peak) or peak <= 0):
        raise ConfigError("peak-tflops-per-gpu must be finite and positive")


def _refuse_used_directory(directory: Path, rank: int) -> None:
    found = [f"{prefix}.rank{rank}.json" for prefix in RECORD_PREFIXES
             if (directory / f"{prefix}.rank{rank}.json").exists()]
    if found:
        raise ConfigError(
            f"Output directory already contains rank {rank} experiment records: "
            f"{', '.join(found)}. Choose a new --debug.output_dir to preserve prior traces "
            "and snapshots.")


def _header(config, session, warmup, profile_mode, profile_detail, runtime_events) -> dict:
    mesh, tc = session.context, config.training
    on_cuda = mesh.device.type == "cuda"
    policy = dict(PRECISION_POLICY_ROLES)
    policy.update(dict.fromkeys(COMPUTE_DTYPE_ROLES, tc.dtype))
    return {
        "engine": "shardtrain_b200",
        "status": "initializing",
        "rank": session.worker.rank,
        "world_size": session.worker.world_size,
        "coordinate": asdict(mesh.coordinate),
        "versions": software_versions(),
        "device": str(mesh.device),
        "device_name": torch.cuda.get_device_name(mesh.device) if on_cuda else "CPU",
        "device_capability": torch.cuda.get_device_capability(mesh.device) if on_cuda else None,
        "attention_backend": "tcgen05 causal GQA kernels (sm_100a executor) or PyTorch SDPA math "
                             "with grouped KV expansion (portable executor)",
        "dtype": tc.dtype,
        "optimizer": tc.optimizer,
        "micro_batch": tc.local_batch_size,
        "global_batch": tc.local_batch_size * tc.accumulation_steps * config.parallel.fsdp_degree,
        "sequence_length": config.model.seq_len,
        "accumulation_steps": tc.accumulation_steps,
        "warmup": warmup,
        "steady_steps_requested": tc.steps,
        "profile_mode": profile_mode,
        "profile_detail": profile_detail,
        "communication_policy": config.runtime.communication_policy,
        "runtime_switches": asdict(config.runtime),
        "runtime_events_enabled": runtime_events,
        "precision_policy": policy,
        "oom": False,
        "nonfinite_loss": False,
        "nonfinite_detected": False,
        "errors": [],
    }


def _timed_step(trainer, device, batch):
    """One optimizer step: (result, host seconds incl. device sync, CUDA-event ms or None)."""
    ids, labels, mask, positions = batch
    span = None
    if device.type == "cuda":
        span = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        span[0].record()
    t0 = time.perf_counter()
    result = trainer.train_step(ids, labels, attention_mask=mask, position_ids=positions)
    if span is not None:
        span[1].record()
        torch.cuda.synchronize(device)
    seconds = time.perf_counter() - t0
    return result, seconds, (span[0].elapsed_time(span[1]) if span is not None else None)


def _finish_record(payload, rows, warmup_rows, device, profile_mode, peak, world_size,
                   runtime, trainer, failed):
    durations = [row["max_rank_seconds"] for row in rows]
    total = sum(durations)
    payload.update({
        "steps": rows,
        "warmup_steps": warmup_rows,
        "steady_steps_completed": len(rows),
        "step_seconds_p50": percentile(durations, 0.50),
        "step_seconds_p95": percentile(durations, 0.95),
        "tokens_per_second": sum(r["valid_tokens"] for r in rows) / total if durations else None,
        "overflow_steps": sum(r["overflow"] for r in rows),
        "warmup_overflow_steps": sum(r["overflow"] for r in warmup_rows),
        "optimizer_updates": sum(not r["overflow"] for r in rows),
        **memory_counters(device),
        "timing_method": "barrier before each step's timer; host wall time of the step including "
                         "the end-of-step device synchronise; max over ranks reduced outside the "
                         "timer; the CUDA-event span covers the whole step timeline; valid "
                         "next-token labels are counted globally over FSDP/SP and exclude "
                         "ignored and final positions",
        "profiling_note": "timings taken with a profile mode other than off are instrumented "
                          "and not comparable; allocator snapshots miss direct CUDA / NCCL / "
                          "peer-memory allocations",
        "benchmark_scope": "synthetic token batch repeated every step",
    })
    if runtime is not None and trainer is not None:
        payload["ownership"] = ownership_audit(runtime, trainer)
        if device.type == "cuda" and not failed:
            payload["pg_order_gpu_waits"] = runtime.comm.gpu_wait_timings()
    source = payload.get("model_source")
    if source is not None and rows:
        payload["performance"] = qwen_performance_summary(
            parameter_numel=source["global_unique_parameter_numel"],
            layers=source["config"]["num_hidden_layers"],
            hidden_size=source["config"]["hidden_size"],
            sequence_length=payload["sequence_length"], global_batch=payload["global_batch"],
            steps=rows, world_size=world_size, peak_tflops_per_gpu=peak,
            profile_mode=profile_mode)


def run(config: Config, *, warmup: int = 0, profile_mode: str = "off",
        profile_detail: str = "low_overhead", runtime_events: bool | None = None,
        peak_tflops_per_gpu: float | None = None) -> dict:
    """Train `config.training.steps` measured optimizer steps after `warmup` unmeasured ones and
    write `benchmark.rank{r}.json`; returns that record.  A failure is written into the record
    (status, errors, oom / nonfinite flags) and then re-raised."""
    _check_arguments(config, warmup, profile_mode, profile_detail, peak_tflops_per_gpu)
    if runtime_events is None:
        runtime_events = profile_mode != "off"
    _refuse_used_directory(Path(config.debug.output_dir), WorkerEnvironment.read().rank)
    with WorkerSession(config, "runtime") as session:
        mesh, tc, rc = session.context, config.training, config.runtime
        device, rank, world = mesh.device, session.worker.rank, session.worker.world_size
        # dropout draws from the global generator; parameter sources carry their own seeds
        torch.manual_seed(tc.seed + rank)
        payload = _header(config, session, warmup, profile_mode, profile_detail, runtime_events)
        rows, warmup_rows = [], []
        runtime = trainer = capture = None
        failure = None
        try:
            try:
                resolve_qwen_compute_dtype(tc.dtype, device)
            except ValueError as exc:
                raise ConfigError(str(exc)) from exc
            record_gpu_topology(session)
            try:
                model = build_qwen_model(config.model, tc.seed)
            except (OSError, ValueError, TypeError) as exc:
                raise ConfigError(f"Cannot construct Qwen model/checkpoint: {exc}") from exc
            payload["model_source"] = describe_model_source(config, model)
            runtime = ShardedRuntime(
                device=device, reshard_after_forward=rc.reshard_after_forward,
                forward_prefetch=rc.forward_prefetch, backward_prefetch=rc.backward_prefetch,
                async_grad_rs=rc.async_grad_rs, communication_policy=rc.communication_policy,
                directory=session.directory, diagnostics_enabled=runtime_events,
                communication_backend=rc.communication_backend,
                retain_parameters=rc.retain_parameters, fused_allgather=rc.fused_allgather,
                wire_dtype=rc.wire_dtype, fused_seq_gather=rc.fused_seq_gather, nvls=rc.nvls, cuda_graphs=rc.cuda_graphs, compute_dtype=tc.dtype,
                device_wait_seconds=config.debug.distributed_timeout_seconds,
            ).register(model, mesh if session.worker.launched else None,
                       sp=config.parallel.sp_enabled)
            trainer = QwenTrainer(model, runtime, tc.lr, dtype=tc.dtype, optimizer=tc.optimizer,
                                  accumulation_steps=tc.accumulation_steps)
            payload["optimizer_hyperparameters"] = trainer.optimizer.defaults
            payload["executor"] = runtime.executor.name
            draw = torch.Generator().manual_seed(tc.seed + mesh.coordinate.fsdp)
            host_ids = torch.randint(model.config.vocab_size,
                                     (tc.local_batch_size * tc.accumulation_steps,
                                      config.model.seq_len), generator=draw)
            payload["input_batch_digest"] = hashlib.sha256(
                json.dumps(host_ids.tolist(), separators=(",", ":")).encode("utf-8")).hexdigest()
            ids = host_ids.to(device)
            batch = (ids, ids.clone(), torch.ones_like(ids),
                     torch.arange(config.model.seq_len, device=device).unsqueeze(0))

            def note(result, row, phase):
                payload["nonfinite_detected"] |= result.overflow
                if not math.isfinite(result.loss):
                    payload["nonfinite_loss"] = True
                    row["loss"] = None
                    raise FloatingPointError(f"Nonfinite Qwen {phase} loss")

            for _ in range(warmup):
                result = trainer.train_step(batch[0], batch[1], attention_mask=batch[2],
                                            position_ids=batch[3])
                warmup_rows.append(asdict(result))
                note(result, warmup_rows[-1], "warmup")
            payload["initialization_and_warmup_memory"] = memory_counters(device)
            runtime.comm.flush_diagnostics(release_events=True)
            if device.type == "cuda":
                torch.cuda.synchronize(device)
                torch.cuda.reset_peak_memory_stats(device)
            capture = ProfileCapture(session.directory, rank, device, mode=profile_mode,
                                     detail=profile_detail)
            capture.start()
            payload["status"] = "running"
            for index in range(tc.steps):
                if dist.is_initialized():
                    dist.barrier()
                result, seconds, gpu_ms = _timed_step(trainer, device, batch)
                row = {**asdict(result), "measured_step": index, "seconds": seconds,
                       "cuda_elapsed_ms": gpu_ms}
                note(result, row, "measured")
                slowest = max_over_ranks(runtime, seconds, world)
                row.update(max_rank_seconds=slowest,
                           tokens_per_second=result.valid_tokens / slowest,
                           **memory_counters(device))
                rows.append(row)
                capture.step(result.step)
                # the timer and the step_complete mark both come before serialisation
                runtime.comm.flush_diagnostics(release_events=True)
                session.logger.info(
                    "qwen step=%d loss=%.8f tokens=%d max_rank_seconds=%.6f overflow=%s",
                    result.step, result.loss, result.valid_tokens, slowest, result.overflow)
            payload["status"] = "completed"
        except BaseException as exc:  # noqa: BLE001 - recorded, then re-raised below
            failure = exc
            text = str(exc).lower()
            payload["status"] = "failed"
            payload["oom"] = isinstance(exc, torch.OutOfMemoryError) or "out of memory" in text
            payload["errors"].append(repr(exc))
            payload["nonfinite_detected"] |= payload["nonfinite_loss"] or "nonfinite" in text
        finally:
            def guarded(label, action):
                nonlocal failure
                try:
                    action()
                except Exception as exc:  # noqa: BLE001
                    payload["errors"].append(f"{label}: {exc!r}")
                    if failure is None:
                        failure, payload["status"] = exc, "failed"

            if capture is not None:
                guarded("profiling", capture.close)
            guarded("summary", lambda: _finish_record(
                payload, rows, warmup_rows, device, profile_mode, peak_tflops_per_gpu, world,
                runtime, trainer, failure is not None))
            if runtime is not None:
                guarded("runtime diagnostics", runtime.comm.close_diagnostics)
            write_json(session.directory / f"benchmark.rank{rank}.json", payload)
        if failure is not None:
            raise failure
        return payload


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0], allow_abbrev=False,
                                     epilog="Config overrides: --section.field value")
    parser.add_argument("--config", default="configs/qwen25_tiny.yaml")
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--profile-mode", choices=["off", "torch", "nsight"], default="off")
    parser.add_argument("--profile-detail", choices=["low_overhead", "full"],
                        default="low_overhead")
    parser.add_argument("--runtime-events", choices=["auto", "on", "off"], default="auto")
    parser.add_argument("--peak-tflops-per-gpu", type=float, default=None)
    args, overrides = parser.parse_known_args(argv)
    try:
        run(load_config(args.config, overrides), warmup=args.warmup,
            profile_mode=args.profile_mode, profile_detail=args.profile_detail,
            runtime_events={"auto": None, "on": True, "off": False}[args.runtime_events],
            peak_tflops_per_gpu=args.peak_tflops_per_gpu)
    except ConfigError as exc:
        parser.error(str(exc))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
