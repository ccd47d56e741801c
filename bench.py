"""Headline benchmark: effective labels/s and mean step ms of Qwen2.5-1.5B training, S512,
global batch 16, gradient accumulation 2, AdamW, bf16 GEMMs with FP32 shards / gradients /
communication, on N GPUs of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W [--strategy F4T2/SP]
    ... --impl reference     # the unmodified reference from baseline/_ref, same metric/config

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events around exactly K steps,
barrier + synchronize on both sides, max over ranks) with the token batch resident on the GPU,
as the reference's own benchmark does; `e2e` repeats the measurement through the public
`QwenTrainer.train_step` API with a host->device copy of the step's tokens from pinned memory and
the device->host read of the step result inside the timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

VALID_LABELS_PER_STEP = 16 * 511          # global batch x (S - 1)
PUBLISHED = {4: {"F4T1": 6543.13, "F2T2/SP": 5370.37}}   # reference README, 4x V100 fp16


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--strategy", default="", help="F{dp}T{tp}[/SP]; default F{gpus}T1")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (not reportable)")
    ap.add_argument("--retain", type=int, default=0, help="runtime.retain_parameters")
    ap.add_argument("--backend", default="auto", choices=["auto", "peer", "nccl"])
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        clocks, reasons, top = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 8:
                continue
            try:
                clocks.append(float(row[0]))
                top = float(row[1])
            except ValueError:
                continue
            for name, value in zip(names, row[4:8]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": top,
                "samples": len(clocks), "reasons": sorted(reasons)}


def qwen15b_dict(args, fsdp, tp, sp, device_backend=("cuda", "nccl")):
    """The benchmark configuration as a plain mapping (shared by both arms)."""
    layers = args.layers or 28
    return ({
        "model": dict(model_type="qwen2", vocab_size=151936, layers=layers, hidden_size=1536,
                      num_heads=12, num_key_value_heads=2, mlp_hidden_size=8960, seq_len=512,
                      rope_theta=1000000.0, tie_word_embeddings=True, rms_norm_eps=1e-6),
        "parallel": dict(fsdp_degree=fsdp, tp_degree=tp, sp_enabled=sp, device=device_backend[0],
                         backend=device_backend[1]),
        "runtime": dict(param_grouping="block", reshard_after_forward=True, forward_prefetch=True,
                        backward_prefetch=True, async_grad_rs=True,
                        communication_policy="stream_ordered",
                        communication_backend=args.backend, retain_parameters=bool(args.retain)),
        "training": dict(dtype="bf16", optimizer="adamw", lr=1e-5, steps=args.steps,
                         local_batch_size=16 // fsdp // 2, accumulation_steps=2, seed=1234),
        "debug": dict(output_dir=f"/tmp/shardtrain_b200_bench_{os.getpid()}",
                      distributed_timeout_seconds=300),
    })


def qwen15b_config(args, fsdp, tp, sp):
    from shardtrain_b200.config import config_from_dict

    return config_from_dict(qwen15b_dict(args, fsdp, tp, sp))


def resolve_strategy(args):
    """(fsdp, tp, sp) from `--strategy F4T2/SP`; default is FSDP over all GPUs."""
    if not args.strategy:
        return args.gpus, 1, False
    text = args.strategy.upper()
    sp = text.endswith("/SP")
    f, t = text[:-3 if sp else None][1:].split("T")
    return int(f), int(t), sp


def run_ours(args):
    import torch
    import torch.distributed as dist

    from shardtrain_b200 import ops
    from shardtrain_b200.launch.bootstrap import WorkerSession
    from shardtrain_b200.models.qwen2_factory import build_qwen_model
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    fsdp, tp, sp = resolve_strategy(args)
    if fsdp * tp != args.gpus:
        raise SystemExit(f"strategy F{fsdp}T{tp} does not match --gpus {args.gpus}")
    config = qwen15b_config(args, fsdp, tp, sp)
    counter = ops.enable_launch_counting()
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
            communication_backend=rc.communication_backend, retain_parameters=rc.retain_parameters,
        ).register(model, mesh if session.worker.launched else None, sp=sp)
        trainer = QwenTrainer(model, runtime, config.training.lr, dtype="bf16", optimizer="adamw",
                              accumulation_steps=config.training.accumulation_steps)
        per_rank = config.training.local_batch_size * config.training.accumulation_steps
        gen = torch.Generator().manual_seed(config.training.seed + mesh.coordinate.fsdp)
        host_ids = torch.randint(model.config.vocab_size, (per_rank, config.model.seq_len),
                                 generator=gen).pin_memory()
        ids = host_ids.to(device)
        multi = session.worker.launched and session.worker.world_size > 1

        def fence():
            if multi:
                dist.barrier()
            torch.cuda.synchronize(device)

        losses = []
        for _ in range(args.warmup):
            losses.append(trainer.train_step(ids).loss)
        # ---- device-timed region: exactly K steps
        sampler = ClockSampler(device.index or 0)
        sampler.start()
        fence()
        launches_before = counter.launches
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(args.steps):
            result = trainer.train_step(ids)
        end.record()
        fence()
        elapsed_ms = begin.elapsed_time(end)
        launches = counter.launches - launches_before
        clocks = sampler.stop()
        losses.append(result.loss)
        # ---- end-to-end region: pinned host tokens in, step result out, every step
        fence()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_ids = host_ids.to(device, non_blocking=True)
            result = trainer.train_step(step_ids)
        fence()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        ops.check_status("bench")
        times = torch.tensor([elapsed_ms, e2e_ms], device=device, dtype=torch.float64)
        if multi:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = times.tolist()
        ms = elapsed_ms / args.steps
        value = VALID_LABELS_PER_STEP * 1000.0 / ms
        strategy = config.parallel.strategy
        published = PUBLISHED.get(args.gpus, {}).get(strategy)
        line = {
            "metric": "effective_labels_per_second", "value": value, "unit": "labels/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": value / published if published else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "impl": "ours",
            "config": {"model": "Qwen2.5-1.5B" + (f" ({args.layers} layers: debug)" if args.layers else ""),
                       "global_batch": 16, "seq_len": 512, "grad_accum": 2, "optimizer": "adamw",
                       "parallelism": strategy, "valid_labels_per_step": VALID_LABELS_PER_STEP,
                       "precision": "bf16 GEMMs; fp32 shards, gradients, communication, AdamW state",
                       "runtime": {"reshard_after_forward": rc.reshard_after_forward,
                                   "forward_prefetch": rc.forward_prefetch,
                                   "backward_prefetch": rc.backward_prefetch,
                                   "async_grad_rs": rc.async_grad_rs,
                                   "communication_policy": rc.communication_policy,
                                   "executor": runtime.executor.name,
                                   "retain_parameters": rc.retain_parameters},
                       "l2": "no explicit flush: each step streams >6 GB of parameters, "
                             "gradients and optimizer state per GPU group, far above the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": VALID_LABELS_PER_STEP * 1000.0 * args.steps / e2e_ms,
                    "unit": "labels/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": host_ids.numel() * host_ids.element_size() * fsdp,
                    "d2h_bytes_per_step": 40 * args.gpus},
            "gpu_launches": launches,
            "loss_first_last": [losses[0] if losses else None, losses[-1]],
            "peak_memory_gib": torch.cuda.max_memory_allocated(device) / 2**30,
        }
        if rank == 0:
            print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
