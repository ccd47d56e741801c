"""Staged acceptance runner: plan a matrix of runs, launch each under a time limit, gate it with
the offline auditors, keep what failed.

    python -m shardtrain_b200.utils.run_matrix --stages groups,flags --max-ranks 4 --dry-run
    python -m shardtrain_b200.utils.run_matrix --stages all --max-ranks 8 --device cuda

What the reference's `scripts/run_matrix.py:138-243` does, restated for this package: stages are
built from a table (mesh list x prefetch / async flag triples), every run gets a directory of its
own with the exact configuration and launch command next to the launcher's output, a run that
exceeds its limit is ended by killing the process group that was started for it (never by name),
and a run only counts as passed when its artifacts pass the gates:

* `groups`     `shardtrain --smoke-groups` on every mesh that fits (one collective per group)
* `flags`      the tiny Qwen2 model through the shard runtime on one mesh, all eight combinations
               of forward prefetch / backward prefetch / asynchronous reduce-scatter; gates:
               the event-log audit, the benchmark-record audit and the measured-payload audit
               of `utils/audit.py`
* `meshes`     the same run with all switches on, on every mesh that fits
* `policies`   conservative against stream_ordered on the largest hybrid mesh that fits; gate: the
               two policies report the same losses

The plan is written to `plan.json` before anything runs (`--dry-run` stops there), every run's
verdict to `summary.json`, and the directories of failed runs are listed at the end.
"""

from __future__ import annotations

import argparse
import itertools
import json
import os
import signal
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

import yaml

from shardtrain_b200.utils.audit import (audit_benchmark, audit_event_logs, audit_volume,
                                         volume_arguments)

ROOT = Path(__file__).resolve().parents[2]
MESHES = [(1, 1), (2, 1), (1, 2), (2, 2), (4, 1), (4, 2), (2, 4), (8, 1)]       # (F, T)
STAGES = ("groups", "flags", "meshes", "policies")
LAUNCHER_VARIABLES = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT",
                      "TORCHELASTIC_USE_AGENT_STORE")


@dataclass
class Case:
    stage: str
    fsdp: int
    tp: int
    flags: tuple[bool, bool, bool]
    policy: str
    entry: str                      # "smoke" | "qwen"
    directory: str = ""
    command: list[str] = field(default_factory=list)

    @property
    def name(self) -> str:
        bits = "".join(str(int(b)) for b in self.flags)
        return f"{self.stage}_F{self.fsdp}T{self.tp}_flags{bits}_{self.policy}"


def largest_hybrid(max_ranks: int) -> tuple[int, int]:
    for mesh in ((4, 2), (2, 2), (1, 2)):
        if mesh[0] * mesh[1] <= max_ranks:
            return mesh
    return (1, 1)


def plan_cases(stages, max_ranks: int) -> list[Case]:
    fits = [m for m in MESHES if m[0] * m[1] <= max_ranks]
    everything_on = (True, True, True)
    cases: list[Case] = []
    for stage in stages:
        if stage == "groups":
            cases += [Case(stage, f, t, (False,) * 3, "conservative", "smoke") for f, t in fits]
        elif stage == "flags":
            f, t = (2, 2) if max_ranks >= 4 else (2, 1) if max_ranks >= 2 else (1, 1)
            cases += [Case(stage, f, t, flags, "stream_ordered", "qwen")
                      for flags in itertools.product((False, True), repeat=3)]
        elif stage == "meshes":
            cases += [Case(stage, f, t, everything_on, "stream_ordered", "qwen") for f, t in fits]
        elif stage == "policies":
            f, t = largest_hybrid(max_ranks)
            cases += [Case(stage, f, t, everything_on, policy, "qwen")
                      for policy in ("conservative", "stream_ordered")]
        else:
            raise ValueError(f"unknown stage {stage!r} (known: {', '.join(STAGES)})")
    return cases


def write_case(case: Case, run_dir: Path, base: dict, device: str, steps: int) -> None:
    """The case's directory, configuration file and launch command."""
    directory = run_dir / case.name
    directory.mkdir(parents=True)
    config = json.loads(json.dumps(base))
    config["parallel"] = dict(fsdp_degree=case.fsdp, tp_degree=case.tp, sp_enabled=case.tp > 1,
                              device=device, backend="nccl" if device == "cuda" else "gloo")
    config["runtime"].update(forward_prefetch=case.flags[0], backward_prefetch=case.flags[1],
                             async_grad_rs=case.flags[2], reshard_after_forward=True,
                             communication_policy=case.policy)
    config["training"]["steps"] = steps
    config["debug"]["output_dir"] = str(directory)
    if case.tp > 1:
        # heads and sequence must divide by T
        config["model"].update(num_heads=8, num_key_value_heads=4, hidden_size=64)
    if case.entry == "smoke":
        # a process-group check needs the mesh and an output directory, nothing else
        config = {"parallel": dict(config["parallel"], sp_enabled=False), "debug": config["debug"]}
    path = directory / "config.yaml"
    path.write_text(yaml.safe_dump(config, sort_keys=False))
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={case.fsdp * case.tp}", "--rdzv-backend=c10d",
               "--rdzv-endpoint=127.0.0.1:0", "--local-addr=127.0.0.1", "--max-restarts=0"]
    if case.entry == "smoke":
        command += ["-m", "shardtrain_b200.train", "--smoke-groups", "--config", str(path)]
    else:
        command += ["-m", "shardtrain_b200.training.qwen2_benchmark", "--config", str(path),
                    "--warmup", "1", "--runtime-events", "on"]
    (directory / "launch_command.json").write_text(json.dumps(command) + "\n")
    case.directory, case.command = str(directory), command


def launch(case: Case, limit: float) -> tuple[int, float]:
    """Run the case in a process group of its own; on expiry that group, and only it, is killed."""
    env = {k: v for k, v in os.environ.items() if k not in LAUNCHER_VARIABLES}
    env["OMP_NUM_THREADS"] = "1"
    env["PYTHONPATH"] = os.pathsep.join(p for p in (str(ROOT), env.get("PYTHONPATH")) if p)
    began = time.monotonic()
    with open(Path(case.directory) / "launcher.log", "w") as log:
        process = subprocess.Popen(case.command, cwd=ROOT, env=env, stdout=log,
                                   stderr=subprocess.STDOUT, start_new_session=True)
        try:
            status = process.wait(timeout=limit)
        except subprocess.TimeoutExpired:
            os.killpg(process.pid, signal.SIGKILL)       # the session leader's pid is the group id
            process.wait(timeout=30)
            status = -signal.SIGKILL
    return status, time.monotonic() - began


def losses_of(directory) -> list[float] | None:
    path = Path(directory) / "benchmark.rank0.json"
    if not path.exists():
        return None
    record = json.loads(path.read_text())
    return [row["loss"] for row in record.get("steps", []) if "loss" in row] or None


def gate(case: Case, status: int, layers: int, tied: bool) -> list[str]:
    """Reasons this run does not pass (empty: it passes)."""
    if status != 0:
        return [f"launcher exit status {status}"]
    directory = Path(case.directory)
    if case.entry == "smoke":
        missing = [r for r in range(case.fsdp * case.tp)
                   if not (directory / f"smoke.rank{r}.json").exists()]
        return [f"no smoke record of ranks {missing}"] if missing else []
    problems = audit_event_logs(directory, fsdp=case.fsdp, tp=case.tp, layers=layers, tied=tied,
                                policy=case.policy)
    problems += audit_benchmark(directory, layers=layers, tied=tied)
    if case.fsdp * case.tp > 1:
        # every micro-step carried what the volume model predicts from this configuration
        problems += audit_volume(directory, **volume_arguments(directory / "config.yaml"))
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--stages", default="all", help=f"comma list of {', '.join(STAGES)} (or all)")
    ap.add_argument("--max-ranks", type=int, default=4)
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    ap.add_argument("--config", default=str(ROOT / "configs" / "qwen25_tiny.yaml"))
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--limit", type=float, default=300.0, help="seconds allowed per run")
    ap.add_argument("--output", default=None, help="directory of this matrix (default: runs/matrix-<time>)")
    ap.add_argument("--dry-run", action="store_true", help="write plan.json and stop")
    args = ap.parse_args(argv)

    stages = STAGES if args.stages == "all" else tuple(s for s in args.stages.split(",") if s)
    base = yaml.safe_load(Path(args.config).read_text())
    run_dir = Path(args.output or ROOT / "runs" / f"matrix-{time.strftime('%Y%m%d-%H%M%S')}")
    run_dir.mkdir(parents=True, exist_ok=False)
    cases = plan_cases(stages, args.max_ranks)
    for case in cases:
        write_case(case, run_dir, base, args.device, args.steps)
    (run_dir / "plan.json").write_text(json.dumps([asdict(c) for c in cases], indent=2))
    print(f"planned {len(cases)} runs in {run_dir}")
    if args.dry_run:
        return 0

    layers, tied = base["model"]["layers"], base["model"].get("tie_word_embeddings", True)
    summary, by_policy = [], {}
    for case in cases:
        status, seconds = launch(case, args.limit)
        problems = gate(case, status, layers, tied)
        if case.stage == "policies" and not problems:
            by_policy[case.policy] = losses_of(case.directory)
        summary.append({"case": case.name, "status": status, "seconds": round(seconds, 1),
                        "passed": not problems, "problems": problems[:20],
                        "directory": case.directory})
        print(f"{'PASS' if not problems else 'FAIL'}  {case.name}  {seconds:.0f}s"
              + ("" if not problems else f"  {problems[0]}"), flush=True)
    if len(by_policy) == 2 and by_policy["conservative"] != by_policy["stream_ordered"]:
        summary.append({"case": "policies_agree", "passed": False, "directory": str(run_dir),
                        "problems": [f"losses differ between policies: {by_policy}"]})
        print("FAIL  policies_agree")
    (run_dir / "summary.json").write_text(json.dumps(summary, indent=2))
    failed = [row for row in summary if not row["passed"]]
    for row in failed:
        print(f"kept for inspection: {row['directory']}")
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
