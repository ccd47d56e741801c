"""`bench.py --impl reference`: the unmodified reference package (installed into `baseline/_ref`
with `pip install --no-index --no-deps --target baseline/_ref`) driven through its own public
API -- `WorkerSession`, `build_qwen_model`, `ShardedRuntime.register`, `QwenTrainer.train_step` --
on the same model, batch, precision and runtime switches as the `ours` arm, and timed by the same
harness (CUDA events around exactly K steps, barrier + synchronize on both sides, max over
ranks; then an end-to-end pass with a pinned host->device copy of the tokens every step).
Nothing of this repository's models, kernels or engine is imported on this path.
"""

from __future__ import annotations

import json
import os
import sys
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args) -> None:
    if not (REF / "sharded_runtime").is_dir():
        unavailable("baseline/_ref is missing: the reference package was not installed")
        return
    sys.path.insert(0, str(REF))
    try:
        _run(args)
    except Exception as exc:  # noqa: BLE001
        unavailable(f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}")


def _measure(args, fsdp, tp, sp) -> dict:
    import torch
    import torch.distributed as dist
    from sharded_runtime.config import config_from_dict
    from sharded_runtime.launch.bootstrap import WorkerSession
    from sharded_runtime.models.qwen2_factory import build_qwen_model
    from sharded_runtime.runtime import ShardedRuntime
    from sharded_runtime.training.qwen2_trainer import QwenTrainer

    import bench

    ours = bench.qwen15b_dict(args, fsdp, tp, sp)
    for key in ("communication_backend", "retain_parameters", "fused_allgather", "wire_dtype",
                "fused_seq_gather", "nvls", "cuda_graphs"):   # fields the reference lacks
        ours["runtime"].pop(key)
    ours["debug"]["output_dir"] = f"/tmp/shardtrain_ref_bench_{os.getpid()}_{fsdp}x{tp}"
    config = config_from_dict(ours)
    with WorkerSession(config, "runtime") as session:
        mesh, rank = session.context, session.worker.rank
        device = mesh.device
        torch.manual_seed(config.training.seed + rank)
        model = build_qwen_model(config.model, config.training.seed)
        rc = config.runtime
        runtime = ShardedRuntime(
            device=device, reshard_after_forward=rc.reshard_after_forward,
            forward_prefetch=rc.forward_prefetch, backward_prefetch=rc.backward_prefetch,
            async_grad_rs=rc.async_grad_rs, communication_policy=rc.communication_policy,
            directory=None, diagnostics_enabled=False,
        ).register(model, mesh, sp=sp)
        trainer = QwenTrainer(model, runtime, config.training.lr, dtype="bf16", optimizer="adamw",
                              accumulation_steps=config.training.accumulation_steps)
        per_rank = config.training.local_batch_size * config.training.accumulation_steps
        gen = torch.Generator().manual_seed(config.training.seed + mesh.coordinate.fsdp)
        host_ids = torch.randint(model.config.vocab_size, (per_rank, config.model.seq_len),
                                 generator=gen).pin_memory()
        ids = host_ids.to(device)
        mask = torch.ones_like(ids)
        positions = torch.arange(config.model.seq_len, device=device).unsqueeze(0)
        multi = session.worker.launched and session.worker.world_size > 1

        def fence():
            if multi:
                dist.barrier()
            torch.cuda.synchronize(device)

        def step(tokens):
            return trainer.train_step(tokens, tokens.clone(), attention_mask=mask, position_ids=positions)

        losses = [step(ids).loss for _ in range(args.warmup)]
        sampler = bench.ClockSampler(device.index or 0)
        sampler.start()
        fence()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(args.steps):
            result = step(ids)
        end.record()
        fence()
        elapsed_ms = begin.elapsed_time(end)
        clocks = sampler.stop()
        losses.append(result.loss)
        fence()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            result = step(host_ids.to(device, non_blocking=True))
        fence()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        times = torch.tensor([elapsed_ms, e2e_ms], device=device, dtype=torch.float64)
        if multi:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = times.tolist()
        out = dict(strategy=f"F{fsdp}T{tp}" + ("/SP" if sp else ""), rank=rank,
                   ms=elapsed_ms / args.steps, e2e_ms=e2e_ms / args.steps, clocks=clocks,
                   losses=[losses[0] if losses else None, losses[-1]],
                   h2d=host_ids.numel() * host_ids.element_size() * fsdp,
                   peak=torch.cuda.max_memory_allocated(device) / 2**30,
                   switches={"reshard_after_forward": rc.reshard_after_forward,
                             "forward_prefetch": rc.forward_prefetch,
                             "backward_prefetch": rc.backward_prefetch,
                             "async_grad_rs": rc.async_grad_rs,
                             "communication_policy": rc.communication_policy},
                   torch=torch.__version__)
        del trainer, runtime, model
        torch.cuda.empty_cache()
    return out


def _run(args) -> None:
    import bench

    fsdp, tp, sp = bench.resolve_strategy(args)
    if fsdp * tp != args.gpus:
        raise SystemExit(f"strategy F{fsdp}T{tp} does not match --gpus {args.gpus}")
    m = _measure(args, fsdp, tp, sp)
    labels = bench.valid_labels(args)
    value = labels * 1000.0 / m["ms"]
    published = bench.PUBLISHED.get(args.gpus, {}).get(m["strategy"])
    line = {
        "metric": "effective_labels_per_second", "value": value, "unit": "labels/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms"],
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / published if published else None,
        "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
        "impl": "reference",
        "config": {"model": bench.MODELS[args.model]["label"]
                            + (f" ({args.layers} layers: debug)" if args.layers else ""),
                   "global_batch": args.global_batch, "seq_len": bench.MODELS[args.model]["seq_len"],
                   "grad_accum": 2, "optimizer": "adamw",
                   "parallelism": m["strategy"], "valid_labels_per_step": labels,
                   "precision": "bf16 autocast GEMMs, math SDPA; fp32 shards, gradients, "
                                "NCCL communication, AdamW(foreach=False) state",
                   "inputs": "token ids + all-ones attention_mask + position_ids",
                   "runtime": m["switches"], "torch": m["torch"],
                   "l2": "no explicit flush: each step streams >6 GB per GPU group"},
        "clocks": m["clocks"],
        "e2e": {"value": labels * 1000.0 / m["e2e_ms"], "unit": "labels/s",
                "ms_per_step": m["e2e_ms"], "h2d_bytes_per_step": m["h2d"],
                "d2h_bytes_per_step": 24 * args.gpus},
        "gpu_launches": 0,
        "loss_first_last": m["losses"],
        "peak_memory_gib": m["peak"],
    }
    hybrid = bench.HYBRID.get(args.gpus) if args.model == "1.5b" else None
    if hybrid is not None and not args.strategy and not args.no_secondary:
        try:
            bench.next_rendezvous()
            h = _measure(args, *hybrid)
            hv = labels * 1000.0 / h["ms"]
            line["secondary"] = {
                "parallelism": h["strategy"], "value": hv, "unit": "labels/s",
                "ms_per_step": h["ms"],
                "e2e": {"value": labels * 1000.0 / h["e2e_ms"], "ms_per_step": h["e2e_ms"],
                        "h2d_bytes_per_step": h["h2d"], "d2h_bytes_per_step": 24 * args.gpus},
                "loss_first_last": h["losses"], "clocks": h["clocks"],
                "vs_baseline": (hv / bench.PUBLISHED[args.gpus][h["strategy"]]
                                if h["strategy"] in bench.PUBLISHED.get(args.gpus, {}) else None),
            }
        except Exception as exc:  # noqa: BLE001 - the primary measurement must still be printed
            line["secondary"] = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}
    if m["rank"] == 0:
        print(json.dumps(line), flush=True)
