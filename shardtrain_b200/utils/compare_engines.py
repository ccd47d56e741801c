"""Compare the `benchmark.rank*.json` records of two runs of the same workload, for instance this
runtime against the PyTorch-native FSDP2 engine or against the reference package
(the job of `scripts/compare_qwen2_engines.py` in the reference).

    python -m shardtrain_b200.utils.compare_engines runs/ours runs/native [--json]

Both directories must describe the same model, batch, sequence length, accumulation and dtype;
the comparison refuses anything else instead of printing a ratio of different workloads.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

SAME = ("global_batch", "sequence_length", "accumulation_steps", "dtype", "optimizer", "world_size")


def load_run(directory) -> dict:
    """Merge the per-rank records of one run: the step time is the slowest rank's."""
    files = sorted(Path(directory).glob("benchmark.rank*.json"))
    if not files:
        raise FileNotFoundError(f"no benchmark.rank*.json under {directory}")
    records = [json.loads(f.read_text(encoding="utf-8")) for f in files]
    first = records[0]
    if any(r.get("status") != "completed" for r in records):
        raise ValueError(f"{directory}: not every rank completed")
    if len(records) != first.get("world_size", len(records)):
        raise ValueError(f"{directory}: {len(records)} records for world size {first.get('world_size')}")
    steps = min(len(r["steps"]) for r in records)
    per_step = [max(r["steps"][i]["max_rank_seconds"] for r in records) for i in range(steps)]
    tokens = [records[0]["steps"][i]["valid_tokens"] for i in range(steps)]
    losses = [records[0]["steps"][i]["loss"] for i in range(steps)]
    return {
        "directory": str(directory),
        "engine": first.get("engine", "unknown"),
        **{key: first.get(key) for key in SAME},
        "steps": steps,
        "mean_step_ms": 1e3 * sum(per_step) / steps,
        "labels_per_second": sum(tokens) / sum(per_step),
        "first_loss": losses[0],
        "last_loss": losses[-1],
        "max_allocated_gib": max((r.get("max_allocated") or 0) for r in records) / 2**30,
    }


def compare(a: dict, b: dict) -> dict:
    different = [key for key in SAME if a.get(key) != b.get(key)]
    if different:
        raise ValueError("the runs are different workloads: " +
                         ", ".join(f"{k}: {a.get(k)} vs {b.get(k)}" for k in different))
    return {
        "a": a,
        "b": b,
        "throughput_ratio_a_over_b": a["labels_per_second"] / b["labels_per_second"],
        "step_time_ratio_b_over_a": b["mean_step_ms"] / a["mean_step_ms"],
        "first_loss_difference": a["first_loss"] - b["first_loss"],
        "last_loss_difference": a["last_loss"] - b["last_loss"],
    }


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("run_a")
    parser.add_argument("run_b")
    parser.add_argument("--json", action="store_true", help="print the comparison as JSON")
    args = parser.parse_args(argv)
    try:
        result = compare(load_run(args.run_a), load_run(args.run_b))
    except (FileNotFoundError, ValueError) as exc:
        parser.error(str(exc))
    if args.json:
        print(json.dumps(result, indent=2))
        return 0
    for tag in ("a", "b"):
        run = result[tag]
        print(f"{tag}: {run['engine']:<16} {run['mean_step_ms']:9.3f} ms/step  "
              f"{run['labels_per_second']:12.1f} labels/s  loss {run['first_loss']:.5f} -> "
              f"{run['last_loss']:.5f}  peak {run['max_allocated_gib']:.2f} GiB  ({run['directory']})")
    print(f"a / b throughput: {result['throughput_ratio_a_over_b']:.3f}x   "
          f"first-step loss difference: {result['first_loss_difference']:+.2e}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
