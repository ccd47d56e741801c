"""Multi-rank save / re-shard check of the checkpoint formats (CPU/gloo under torchrun).

`--mode save`: train two AdamW steps on the mesh, write the full (canonical) export and the
sharded one.  `--mode load`: build the model on *this* mesh from the full export, re-shard the
optimizer moments, report the reconstructed canonical state and the loss of one more step on a
fixed global batch, so that runs on different F can be compared."""
import argparse
import json
import logging
from pathlib import Path

import torch

from shardtrain_b200.config import ParallelConfig
from shardtrain_b200.distributed.context import DistributedContext, WorkerEnvironment
from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
from shardtrain_b200.models.qwen2_checkpoint import QwenCheckpoint, save_safetensors
from shardtrain_b200.runtime.checkpoint import (
    full_state_dict, load_full_optimizer, load_sharded, save_full, save_sharded,
)
from shardtrain_b200.runtime.engine import ShardedRuntime
from shardtrain_b200.training.qwen2_trainer import QwenTrainer

CFG = dict(vocab_size=256, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
           num_attention_heads=4, num_key_value_heads=2)
GLOBAL_BATCH, SEQ = 4, 16


def batch_for(step, fsdp_rank, fsdp_degree):
    ids = torch.randint(0, CFG["vocab_size"], (GLOBAL_BATCH, SEQ),
                        generator=torch.Generator().manual_seed(50 + step))
    per = GLOBAL_BATCH // fsdp_degree
    return ids[fsdp_rank * per:(fsdp_rank + 1) * per]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    ap.add_argument("--mode", choices=["save", "load", "load_sharded"], required=True)
    ap.add_argument("--fsdp", type=int, default=1)
    a = ap.parse_args()
    worker = WorkerEnvironment.read()
    root = Path(a.dir)
    par = ParallelConfig(a.fsdp, 1, False, "cpu", "gloo")
    with DistributedContext(par, worker, 60, logging.getLogger(f"c{worker.rank}")) as ctx:
        mesh = ctx if worker.launched else None
        model = Qwen2CausalLM(Qwen2ModelConfig(**CFG), device="meta", dtype=torch.float32)
        model._qwen_seed = 11
        if a.mode == "load":
            model._qwen_weight_source = QwenCheckpoint(root / "full")
        rt = ShardedRuntime(device="cpu").register(model, mesh)
        tr = QwenTrainer(model, rt, lr=1e-3, optimizer="adamw")
        f = ctx.coordinate.fsdp
        if a.mode == "save":
            for step in range(2):
                tr.train_step(batch_for(step, f, a.fsdp))
            save_full(rt, root / "full", tr.optimizer)
            save_sharded(rt, root / "sharded", tr.optimizer, trainer=tr)
        elif a.mode == "load":
            load_full_optimizer(rt, root / "full", tr.optimizer)
        else:
            meta = load_sharded(rt, root / "sharded", tr.optimizer, trainer=tr)
            assert tr.step_id == 2 and rt.step_id == meta["runtime_step"]
        state = full_state_dict(rt, tr.optimizer)
        loss = tr.train_step(batch_for(2, f, a.fsdp)).loss
        if worker.rank == 0:
            tag = f"{a.mode}.f{a.fsdp}"
            save_safetensors(root / f"state.{tag}.safetensors", {k: v.cpu() for k, v in state.items()})
            (root / f"loss.{tag}.json").write_text(json.dumps({"loss": loss}))


if __name__ == "__main__":
    main()
