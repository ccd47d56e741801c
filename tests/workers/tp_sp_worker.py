"""Legacy synchronous TP / TP+SP path on gloo: the converted toy stack trained with `Trainer`
must follow the unsharded model trained on the same data (CPU, under torchrun)."""
import argparse
import copy
import json
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200.config import ModelConfig
from shardtrain_b200.models.reference import build_reference_model, synthetic_batch
from shardtrain_b200.parallel.model import parallelize_tp_sp
from shardtrain_b200.training.trainer import ReferenceTrainer, Trainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--sp", type=int, default=0)
    a = ap.parse_args()
    dist.init_process_group("gloo")
    rank, degree = dist.get_rank(), dist.get_world_size()
    group = dist.new_group(list(range(degree)), backend="gloo")
    cfg = ModelConfig(layers=2, hidden_size=32, num_heads=4, mlp_hidden_size=64, seq_len=8)
    dense = build_reference_model(cfg, 1234)
    # every other rank starts from different values: the conversion must broadcast rank 0's
    model = copy.deepcopy(dense) if rank == 0 else build_reference_model(cfg, 99 + rank)
    plan = parallelize_tp_sp(model, group, sp=bool(a.sp))
    trainer, reference = Trainer(model, 0.05, 2, tp_plan=plan), ReferenceTrainer(dense, 0.05, 2)
    rows = []
    for step in range(3):
        batch = synthetic_batch(cfg, 4, 500 + step)
        got = trainer.train_step(plan.input_for_rank(batch))
        want = reference.train_step(batch)
        rows.append(dict(loss=got.loss, ref=want.loss))
    full = plan.global_parameters()
    worst = max((full[n] - p.detach()).abs().max().item() for n, p in dense.named_parameters())
    column = plan.partitions["0.attention.q_proj.weight"]
    Path(a.out).mkdir(parents=True, exist_ok=True)
    (Path(a.out) / f"tp.rank{rank}.json").write_text(json.dumps(dict(
        rows=rows, worst=worst, column_dim=column.dim, heads=model[0].attention.num_heads,
        local_rows=model[0].attention.q_proj.weight.shape[0])))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
