"""torchrun worker: train the tiny Qwen2 for a few steps on an F x T mesh and compare losses,
reconstructed parameters and event counts against an unsharded single-process model."""
import argparse
import json
import logging
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200.config import ParallelConfig
from shardtrain_b200.distributed.context import DistributedContext, WorkerEnvironment
from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
from shardtrain_b200.runtime.engine import ShardedRuntime
from shardtrain_b200.training.qwen2_trainer import QwenTrainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--fsdp", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--sp", type=int, default=0)
    ap.add_argument("--flags", default="000")
    ap.add_argument("--policy", default="conservative")
    ap.add_argument("--reshard", type=int, default=1)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--tied", type=int, default=1)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--mismatch", type=int, default=0)
    ap.add_argument("--shape", default="tiny", choices=["tiny", "tiny4", "d128", "d128tp"])
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--optimizer", default="adamw")
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--fused-allgather", default="auto")
    ap.add_argument("--wire", default="bf16")
    ap.add_argument("--seq-pull", type=int, default=0)
    ap.add_argument("--nvls", default="off")
    ap.add_argument("--inject-inf-rank", type=int, default=-1,
                    help="this rank poisons one shard gradient with inf in step 1 (host-side injection)")
    ap.add_argument("--delay-rank", type=int, default=-1,
                    help="this rank sleeps 50 ms on the host before every step (rank skew)")
    a = ap.parse_args()
    worker = WorkerEnvironment.read()
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    logger = logging.getLogger(f"w{worker.rank}")
    backend = "gloo" if a.device == "cpu" else "nccl"
    par = ParallelConfig(a.fsdp, a.tp, bool(a.sp), a.device, backend)
    if a.device == "cuda" and a.policy == "stream_ordered" and worker.world_size > 1:
        from shardtrain_b200.distributed.nccl_ordering import prepare_nccl_launch_order
        prepare_nccl_launch_order()   # what WorkerSession does for the NCCL path
    with DistributedContext(par, worker, 60, logger) as ctx:
        if a.shape == "d128":   # head_dim 128: the shape class of the sm_100a kernels
            cfg = Qwen2ModelConfig(vocab_size=2048, hidden_size=256, intermediate_size=512,
                                   num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                                   tie_word_embeddings=bool(a.tied))
        elif a.shape == "d128tp":   # head_dim 128 with 2 KV heads: divisible by TP 2
            cfg = Qwen2ModelConfig(vocab_size=2048, hidden_size=512, intermediate_size=512,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                   tie_word_embeddings=bool(a.tied))
        elif a.shape == "tiny4":   # 4 KV heads: divisible by TP 4
            cfg = Qwen2ModelConfig(vocab_size=1024, hidden_size=64, intermediate_size=128,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                                   tie_word_embeddings=bool(a.tied))
        else:
            cfg = Qwen2ModelConfig(vocab_size=1024, hidden_size=64, intermediate_size=128,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                   tie_word_embeddings=bool(a.tied))
        vocab, seq = cfg.vocab_size, (256 if a.shape.startswith("d128") else 64)
        torch.manual_seed(7 + (worker.rank if a.mismatch else 0))
        dense = Qwen2CausalLM(cfg)
        import copy
        model = copy.deepcopy(dense)
        fp, bp, ar = (c == "1" for c in a.flags)
        rt = ShardedRuntime(device=ctx.device, reshard_after_forward=bool(a.reshard),
                            forward_prefetch=fp, backward_prefetch=bp, async_grad_rs=ar,
                            communication_policy=a.policy, directory=out,
                            communication_backend=a.backend, compute_dtype=a.dtype,
                            fused_allgather=a.fused_allgather, wire_dtype=a.wire,
                            fused_seq_gather=bool(a.seq_pull), nvls=a.nvls)
        rt.register(model, ctx, sp=bool(a.sp))
        lr = 1e-3 if a.optimizer == "adamw" else 0.05
        tr = QwenTrainer(model, rt, lr=lr, optimizer=a.optimizer, accumulation_steps=a.accum,
                         dtype=a.dtype)
        dense = dense.to(ctx.device)
        opt = (torch.optim.AdamW if a.optimizer == "adamw" else torch.optim.SGD)(dense.parameters(), lr=lr)
        batch = 2 * a.accum
        rows = []
        if a.inject_inf_rank >= 0:
            finalize = rt.finalize_backward

            def poisoned(*args, **kwargs):
                if worker.rank == a.inject_inf_rank and tr.step_id == 1:
                    rt.grad_arena[3] = float("inf")
                return finalize(*args, **kwargs)

            rt.finalize_backward = poisoned
        for step in range(a.steps):
            gen = torch.Generator().manual_seed(100 + step)
            # every FSDP coordinate trains on its own batch; TP ranks of a replica share it
            all_ids = torch.randint(0, vocab, (a.fsdp, batch, seq), generator=gen)
            ids = all_ids[ctx.coordinate.fsdp].to(ctx.device)
            if worker.rank == a.delay_rank:
                import time
                time.sleep(0.05)
            try:
                res = tr.train_step(ids)
            except RuntimeError as exc:
                if a.inject_inf_rank < 0:
                    raise
                # every rank must refuse the poisoned step, and the runtime must stay failed
                refused_again = False
                try:
                    tr.train_step(ids)
                except RuntimeError:
                    refused_again = True
                (out / f"failure.rank{worker.rank}.json").write_text(json.dumps(dict(
                    step=step, error=str(exc), failed=rt.failed, refused_again=refused_again)))
                return
            opt.zero_grad()
            flat = all_ids.reshape(-1, seq).to(ctx.device)
            with torch.autocast(ctx.device.type, dtype=torch.bfloat16, enabled=a.dtype == "bf16"):
                ref = dense(flat, labels=flat)
            ref.loss.backward()
            opt.step()
            rows.append(dict(step=step, loss=res.loss, ref=ref.loss.item(), valid=res.valid_tokens))
        full = rt.reconstruct_tp_local()
        err, errs = 0.0, {}
        for name, p in dense.named_parameters():
            part = rt.qwen_partitions[name].local_slice(p.detach()).cpu()
            e = (full[name].cpu() - part).abs().max().item()
            errs[name] = e
            err = max(err, e)
        events = {}
        for e in rt.comm.events:
            events[e["event_type"]] = events.get(e["event_type"], 0) + 1
        kinds = {}
        for t in rt.comm.tickets:
            kinds[t.kind] = kinds.get(t.kind, 0) + 1
        seq = [(t.pg_id, t.kind, t.unit_id, t.phase) for t in rt.comm.tickets]
        shard_ok = all(p.ndim == 1 and p.dtype == torch.float32 for p in model.parameters())
        (out / f"result.rank{worker.rank}.json").write_text(json.dumps(dict(
            rows=rows, param_err=err, events=events, kinds=kinds, seq=seq, shard_ok=shard_ok,
            live=len(rt.comm.live_buffers), names=[n for n, _ in model.named_parameters()][:4],
            units=len(rt.units), leaves=len(rt.registry), errs=errs,
            nvls=bool(getattr(rt.fused, "nvls_active", False)),
            nvls_refusal=getattr(getattr(rt.fused, "reduce_peer", None), "multicast_refusal", None))))
        rt.comm.flush_diagnostics()
        if ctx.device.type == "cuda":
            from shardtrain_b200 import ops
            torch.cuda.synchronize()
            ops.check_status("worker")


if __name__ == "__main__":
    main()
