"""Where one optimizer step spends its time: a kineto capture of a single training step of the
Qwen2.5 benchmark workload, summarised on rank 0 as text (no trace viewer needed).

    python -m shardtrain_b200.ops.profile_step --global-batch 16
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m shardtrain_b200.ops.profile_step --global-batch 4          # the 8-GPU per-rank shape on 2 GPUs

Printed: the step's span, the union of all kernel intervals, the kernel time per stream (compute,
parameter gather, gradient reduce-scatter), the largest kernels by total time, and the idle gaps
of the compute stream grouped by the kernel that ended them (a gap before a layer's first kernel
is a wait for that layer's parameters; one before the embedding lookup is a micro-step boundary).
Times under a profiler are for shares, not for reporting step times.
"""

from __future__ import annotations

import argparse
import json
import os
import tempfile


def short(name: str) -> str:
    return (name.replace("(anonymous namespace)::", "").replace("void ", "").replace("stb::", "")
            .split("(")[0][:56])


def summarise(trace_path: str, top: int = 16) -> dict:
    events = json.load(open(trace_path))["traceEvents"]
    kernels = sorted((e for e in events if e.get("cat") == "kernel"), key=lambda e: e["ts"])
    if not kernels:
        return {"kernels": 0}
    begin = kernels[0]["ts"]
    end = max(e["ts"] + e["dur"] for e in kernels)
    busy, lo, hi = 0.0, None, None
    for e in kernels:
        s, t = e["ts"], e["ts"] + e["dur"]
        if hi is None or s > hi:
            busy += (hi - lo) if hi is not None else 0.0
            lo, hi = s, t
        else:
            hi = max(hi, t)
    busy += hi - lo
    by_name: dict[str, list] = {}
    by_stream: dict[int, list] = {}
    for e in kernels:
        entry = by_name.setdefault(short(e["name"]), [0, 0.0])
        entry[0] += 1
        entry[1] += e["dur"]
        by_stream.setdefault(e["args"].get("stream"), []).append(e)
    compute = max(by_stream.values(), key=len)          # the stream with the most launches
    gaps: dict[str, list] = {}
    previous_end = None
    for e in compute:
        if previous_end is not None and e["ts"] - previous_end > 15:
            entry = gaps.setdefault(short(e["name"]), [0, 0.0])
            entry[0] += 1
            entry[1] += e["ts"] - previous_end
        previous_end = e["ts"] + e["dur"]
    return {
        "kernels": len(kernels),
        "span_ms": (end - begin) / 1e3,
        "busy_union_ms": busy / 1e3,
        "kernel_sum_ms": sum(e["dur"] for e in kernels) / 1e3,
        "streams": sorted(({"launches": len(v), "kernel_ms": sum(e["dur"] for e in v) / 1e3}
                           for v in by_stream.values()), key=lambda r: -r["launches"]),
        "top_kernels": [{"name": n, "launches": c, "total_ms": d / 1e3, "mean_us": d / c}
                        for n, (c, d) in sorted(by_name.items(), key=lambda kv: -kv[1][1])[:top]],
        "compute_stream_gaps_over_15us": {
            "total_ms": sum(d for _, d in gaps.values()) / 1e3,
            "before": [{"kernel": n, "count": c, "total_ms": d / 1e3}
                       for n, (c, d) in sorted(gaps.items(), key=lambda kv: -kv[1][1])[:10]]},
    }


def main(argv=None) -> int:
    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    from shardtrain_b200.config import config_from_dict
    from shardtrain_b200.launch.bootstrap import WorkerSession
    from shardtrain_b200.models.qwen2_factory import build_qwen_model
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--global-batch", type=int, default=16)
    ap.add_argument("--tp", type=int, default=1, help="TP degree (with sequence parallelism)")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--output", default=None, help="also write the summary (JSON) to this file")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--nvls", default="off", choices=["auto", "off"])
    ap.add_argument("--fused-allgather", default="auto", choices=["auto", "on", "off"])
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    fsdp = world // args.tp
    config = config_from_dict({
        "model": dict(model_type="qwen2", layers=args.layers, seq_len=512, rope_theta=1000000.0,
                      rms_norm_eps=1e-6, vocab_size=151936, hidden_size=1536, num_heads=12,
                      num_key_value_heads=2, mlp_hidden_size=8960, tie_word_embeddings=True),
        "parallel": dict(fsdp_degree=fsdp, tp_degree=args.tp, sp_enabled=args.tp > 1, device="cuda",
                         backend="nccl"),
        "runtime": dict(param_grouping="block", reshard_after_forward=True, forward_prefetch=True,
                        backward_prefetch=True, async_grad_rs=True,
                        communication_policy="stream_ordered", nvls=args.nvls,
                        fused_allgather=args.fused_allgather, cuda_graphs=not args.no_graphs),
        "training": dict(dtype="bf16", optimizer="adamw", lr=1e-5, steps=1,
                         local_batch_size=args.global_batch // fsdp // 2, accumulation_steps=2, seed=1234),
        "debug": dict(output_dir=os.path.join(tempfile.gettempdir(), f"profile_step_{os.getpid()}"),
                      distributed_timeout_seconds=120),
    })
    with WorkerSession(config, "runtime") as session:
        mesh, rank = session.context, session.worker.rank
        rc = config.runtime
        model = build_qwen_model(config.model, config.training.seed)
        runtime = ShardedRuntime(
            device=mesh.device, reshard_after_forward=True, forward_prefetch=True,
            backward_prefetch=True, async_grad_rs=True, communication_policy="stream_ordered",
            diagnostics_enabled=False, compute_dtype="bf16", device_wait_seconds=10,
            fused_allgather=rc.fused_allgather, nvls=rc.nvls, cuda_graphs=rc.cuda_graphs,
        ).register(model, mesh if session.worker.launched else None, sp=args.tp > 1)
        trainer = QwenTrainer(model, runtime, 1e-5, dtype="bf16", optimizer="adamw", accumulation_steps=2)
        ids = torch.randint(0, 151936, (args.global_batch // fsdp, 512), device=mesh.device)
        mask, positions = torch.ones_like(ids), torch.arange(512, device=mesh.device).unsqueeze(0)

        def step():
            trainer.train_step(ids, ids, attention_mask=mask, position_ids=positions)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        if session.worker.launched and world > 1:
            dist.barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        if rank == 0:
            path = os.path.join(tempfile.gettempdir(), f"profile_step_{os.getpid()}.json")
            prof.export_chrome_trace(path)
            summary = summarise(path)
            os.unlink(path)
            summary["mesh"] = {"fsdp": fsdp, "tp": args.tp, "global_batch": args.global_batch,
                               "cuda_graphs": rc.cuda_graphs, "nvls": rc.nvls}
            print(json.dumps(summary, indent=1))
            if args.output:
                with open(args.output, "w") as out:
                    json.dump(summary, out, indent=1)
        runtime.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
