"""Offline acceptance checks over a run's artefacts.

Two auditors, both returning a list of human-readable violations (empty = accepted):

* `audit_event_logs(directory, fsdp=, tp=, layers=, tied=)` reads every
  `runtime_events.rank{r}.jsonl` of a run and checks the runtime's behavioural contract on it:
  communicator membership and gap-free per-communicator sequence numbers, issue -> work ->
  consumable order of every collective, buffer lifetimes (allocated once, retired once, nothing
  live at `optimizer_ready` / `step_end`), materialisation / reduction / commit counts per
  micro-step, the ordering policy's edges (completion edges under `conservative`, none under
  `stream_ordered`), the gradient-dispatch prefetch order, and equality of every communicator's
  issue sequence across its members.  The rules are those the reference enforces with
  `scripts/audit_qwen_gpu_acceptance.py:172-392` and `scripts/run_matrix.py:55-79`.
* `audit_benchmark(directory, ...)` gates `benchmark.rank{r}.json`: completed, finite, one
  optimizer update per step, ownership block (no live buffers or leases, stable shard identity,
  unit and leaf counts, FP32 masters, gradient bytes = parameter bytes, optimizer state for
  every leaf), `valid_tokens` = F x local batch x accumulation x (S - 1) on every step, switches
  echoed, and (step, overflow, loss scale, tokens, loss) identical across ranks
  (`scripts/run_qwen_v100_workload.py:369-522, 594-615` of the reference).

    python -m shardtrain_b200.utils.audit events RUN_DIR --fsdp 2 --tp 2 --layers 28
    python -m shardtrain_b200.utils.audit benchmark RUN_DIR --layers 28
"""

from __future__ import annotations

import argparse
import json
import math
from collections import Counter, defaultdict
from pathlib import Path


# ---------------------------------------------------------------------------- event logs
def read_events(directory) -> dict[int, list[dict]]:
    logs = {}
    for path in sorted(Path(directory).glob("runtime_events.rank*.jsonl")):
        rank = int(path.name.split("rank")[1].split(".")[0])
        logs[rank] = [json.loads(line) for line in path.read_text().splitlines() if line.strip()]
    return logs


def expected_members(role: str, rank: int, fsdp: int, tp: int) -> list[int]:
    """Ranks of the communicator `role` that contains `rank` (rank = f * tp + t)."""
    f, t = divmod(rank, tp)
    if role.startswith("tp"):
        return [f * tp + i for i in range(tp)]
    if role.startswith("fsdp"):
        return [i * tp + t for i in range(fsdp)]
    return list(range(fsdp * tp))


class _RankAudit:
    def __init__(self, rank, rows, fsdp, tp, layers, tied, policy):
        self.rank, self.rows, self.fsdp, self.tp = rank, rows, fsdp, tp
        self.layers, self.tied, self.policy = layers, tied, policy
        self.problems: list[str] = []

    def fail(self, text):
        self.problems.append(f"rank {self.rank}: {text}")

    # -- communicators -------------------------------------------------------------------
    def communicators(self):
        last_seq: dict[str, int] = {}
        for row in self.rows:
            if row["event_type"] != "collective_issue":
                continue
            pg, seq = row["pg_id"], row["pg_local_seq"]
            if seq != last_seq.get(pg, -1) + 1:
                self.fail(f"{pg} sequence jumps from {last_seq.get(pg, -1)} to {seq} (op {row['op_id']})")
            last_seq[pg] = seq
            members = row.get("group_members") or []
            if len(members) > 1 and list(members) != expected_members(pg, self.rank, self.fsdp, self.tp):
                self.fail(f"{pg} op {row['op_id']} lists members {members}")

    # -- issue -> work -> consumable -------------------------------------------------------
    def collective_order(self):
        stage: dict[int, int] = {}
        for row in self.rows:
            op, kind = row.get("op_id"), row["event_type"]
            if kind == "collective_issue":
                if op in stage:
                    self.fail(f"op {op} issued twice")
                stage[op] = 0
            elif kind == "work_issued":
                if stage.get(op) != 0:
                    self.fail(f"op {op}: work_issued without a preceding collective_issue")
                stage[op] = 1
            elif kind == "collective_consumer_ready":
                if stage.get(op, -1) < 1:
                    self.fail(f"op {op}: consumable before its work was issued")
                stage[op] = 2
        open_ops = [op for op, s in stage.items() if s < 2]
        if open_ops:
            self.fail(f"collectives never consumed: {open_ops[:8]}")

    # -- buffers ---------------------------------------------------------------------------
    def buffers(self):
        live: dict[int, str] = {}
        seen: set[int] = set()
        for row in self.rows:
            kind, buf = row["event_type"], row.get("buffer_id")
            if kind == "buffer_allocate":
                if buf in seen:
                    self.fail(f"buffer {buf} allocated twice")
                seen.add(buf)
                live[buf] = row.get("buffer_kind") or row.get("kind") or "?"
            elif kind == "buffer_retire":
                if buf not in live:
                    self.fail(f"buffer {buf} retired without being live")
                live.pop(buf, None)
            elif kind in ("optimizer_ready", "step_end") and live:
                self.fail(f"{len(live)} live buffer(s) at {kind} of step {row['step_id']}: "
                          f"{sorted(live)[:6]}")
            for key in ("input_buffer_ids", "output_buffer_ids"):
                if kind == "collective_issue":
                    for ref in row.get(key) or []:
                        if ref not in live:
                            self.fail(f"op {row['op_id']} references buffer {ref} that is not live")

    # -- per micro-step counts -----------------------------------------------------------------
    def step_counts(self):
        by_step: dict[int, list[dict]] = defaultdict(list)
        for row in self.rows:
            if row["step_id"] >= 0:
                by_step[row["step_id"]].append(row)
        units = self.layers + 2 + (0 if self.tied else 1)
        leaves = 12 * self.layers + 2 + (0 if self.tied else 1)
        for step, rows in sorted(by_step.items()):
            kinds = Counter(r["event_type"] for r in rows)
            if not kinds.get("step_end") and not kinds.get("optimizer_ready"):
                continue       # an unfinished trailing step
            gathers = [r for r in rows if r["event_type"] == "materialize_issue"]
            retained_last = {0, self.layers + 1} if self.tied else {units - 1}
            expected = 2 * units - len(retained_last)
            if len(gathers) != expected:
                self.fail(f"step {step}: {len(gathers)} materialisations, expected {expected}")
            for r in gathers:
                if r["phase"] == "BWD" and r["unit_id"] in retained_last:
                    self.fail(f"step {step}: unit {r['unit_id']} re-gathered in backward")
            reduced = Counter(r["unit_id"] for r in rows if r["event_type"] == "unit_grads_ready")
            if sorted(reduced) != list(range(units)) or set(reduced.values()) != {1}:
                self.fail(f"step {step}: unit reductions {dict(reduced)}")
            commits = Counter(r.get("param_id") for r in rows if r["event_type"] == "leaf_grad_committed")
            if len(commits) != leaves or set(commits.values()) != {1}:
                self.fail(f"step {step}: {len(commits)} leaves committed "
                          f"({sum(commits.values())} commits), expected {leaves} once each")
            if kinds.get("optimizer_ready", 0) != 1:
                self.fail(f"step {step}: {kinds.get('optimizer_ready', 0)} optimizer_ready events")
            if kinds.get("step_end", 0) > 1:
                self.fail(f"step {step}: {kinds['step_end']} step_end events")

    # -- ordering policy --------------------------------------------------------------------------
    def policy_edges(self):
        if self.policy is None:
            return
        pg_order = [r for r in self.rows if r["event_type"] == "dependency_edge"
                    and r.get("dependency_type") == "PG_ORDER"]
        launch = [r for r in self.rows if r["event_type"] == "collective_launch_order"]
        if self.policy == "stream_ordered":
            if pg_order:
                self.fail(f"stream_ordered run carries {len(pg_order)} PG_ORDER completion edges")
            for r in launch:
                if r.get("gpu_completion_dependency"):
                    self.fail(f"op {r['op_id']}: launch-order edge with a GPU completion dependency")
        elif launch:
            self.fail("conservative run carries host launch-order edges")

    # -- gradient-dispatch prefetch -----------------------------------------------------------------
    def dispatch_order(self):
        """Owner U (>= 2) issues both buckets, then the gather of unit U - 2, and only then
        consumes its reductions."""
        by_step: dict[int, list[dict]] = defaultdict(list)
        for row in self.rows:
            by_step[row["step_id"]].append(row)
        for step, rows in by_step.items():
            tokens = [r for r in rows if r["event_type"] == "backward_prefetch_token"]
            for token in tokens:
                owner = token.get("gradient_owner")
                if owner is None:
                    continue
                index = rows.index(token)
                before = [r for r in rows[:index] if r.get("unit_id") == owner and r["phase"] == "BWD"]
                after = [r for r in rows[index:] if r.get("unit_id") == owner and r["phase"] == "BWD"]
                issued = [r for r in before if r["event_type"] == "gradient_bucket_issued"]
                consumed_early = [r for r in before if r["event_type"] == "gradient_bucket_consumed"]
                consumed_late = [r for r in after if r["event_type"] == "gradient_bucket_consumed"]
                if not issued or consumed_early or len(consumed_late) != len(issued):
                    self.fail(f"step {step}: dispatch of owner U{owner} is not between the issue "
                              "and the consumption of its reductions")
                if token.get("target_unit") != owner - 2:
                    self.fail(f"step {step}: owner U{owner} dispatched U{token.get('target_unit')}")

    def run(self):
        self.communicators()
        self.collective_order()
        self.buffers()
        self.step_counts()
        self.policy_edges()
        self.dispatch_order()
        return self.problems


def issue_sequences(rows) -> dict[str, list[tuple]]:
    sequences: dict[str, list[tuple]] = defaultdict(list)
    for r in rows:
        if r["event_type"] == "collective_issue":
            sequences[r["pg_id"]].append((r.get("op_kind"), r.get("numel"), r.get("dtype"),
                                          r.get("unit_id"), r.get("phase"), r.get("step_id"),
                                          tuple(r.get("input_shape") or ()),
                                          tuple(r.get("output_shape") or ())))
    return sequences


def audit_event_logs(directory, *, fsdp: int, tp: int, layers: int, tied: bool = True,
                     policy: str | None = None) -> list[str]:
    logs = read_events(directory)
    if sorted(logs) != list(range(fsdp * tp)):
        return [f"event logs of ranks {sorted(logs)} found, expected {fsdp * tp} ranks"]
    problems: list[str] = []
    for rank, rows in logs.items():
        problems += _RankAudit(rank, rows, fsdp, tp, layers, tied, policy).run()
    # every member of a communicator issued the same sequence
    sequences = {rank: issue_sequences(rows) for rank, rows in logs.items()}
    for rank in logs:
        for role in sequences[rank]:
            members = expected_members(role, rank, fsdp, tp)
            first = members[0]
            if rank != first and sequences[rank][role] != sequences[first].get(role):
                mine, theirs = sequences[rank][role], sequences[first].get(role, [])
                where = next((i for i, (a, b) in enumerate(zip(mine, theirs)) if a != b),
                             min(len(mine), len(theirs)))
                problems.append(f"{role} communicator {members}: rank {rank} diverges from rank "
                                f"{first} at position {where}")
    return problems


# ---------------------------------------------------------------------------- benchmark artefacts
# kinds the event log uses for each role (gloo computes a reduce-scatter as all-reduce + slice)
VOLUME_KINDS = {"fsdp_ag": {"fsdp_ag"}, "fsdp_rs": {"fsdp_rs", "fsdp_rs_math_allreduce"},
                "sp_ag": {"sp_ag"}, "sp_rs": {"sp_rs", "sp_rs_math_allreduce"},
                "tp_replicated_allreduce": {"tp_norm_allreduce"}}


def audit_volume(directory, model: dict, *, fsdp: int, tp: int, sp: bool, local_batch: int) -> list[str]:
    """Measured payload against the model: in every micro-step of every rank, the collectives of
    each role are as many, and carry as many elements, as `comm_volume.microstep_payload` predicts
    from the configuration alone (the reference's "predicted vs. measured payload" table,
    reports/fsdp_interview_sections/04_communication_volume.md:84-95)."""
    from shardtrain_b200.utils.comm_volume import microstep_payload

    want = microstep_payload(model, fsdp=fsdp, tp=tp, sp=sp, local_batch=local_batch)
    if fsdp == 1:
        want.pop("fsdp_ag"), want.pop("fsdp_rs")        # a singleton group issues nothing
    problems = []
    for rank, rows in read_events(directory).items():
        seen: dict[tuple[int, str], list[int]] = defaultdict(lambda: [0, 0])
        for r in rows:
            if r["event_type"] != "collective_issue" or r.get("step_id", -1) < 0:
                continue
            if r.get("phase") not in ("FWD", "BWD"):
                continue
            for role, kinds in VOLUME_KINDS.items():
                if r.get("kind") in kinds:
                    shape = r.get("output_shape") if role.endswith("_ag") else r.get("input_shape")
                    elements = 1
                    for extent in shape or [r.get("numel", 0)]:
                        elements *= extent
                    entry = seen[(r["step_id"], role)]
                    entry[0] += 1
                    entry[1] += elements
        steps = sorted({step for step, _ in seen})
        for step in steps:
            for role, expect in want.items():
                count, elements = seen.get((step, role), (0, 0))
                low = expect.get("count", expect.get("count_min"))
                high = expect.get("count", expect.get("count_max"))
                if not low <= count <= high:
                    problems.append(f"rank {rank} step {step}: {count} {role} collectives, "
                                    f"expected {low}" + ("" if low == high else f"..{high}"))
                if elements != expect["elements"]:
                    problems.append(f"rank {rank} step {step}: {role} carried {elements} elements, "
                                    f"the model predicts {expect['elements']}")
        if not steps:
            problems.append(f"rank {rank}: no micro-step with collectives found")
    return problems


def volume_arguments(config_path) -> dict:
    """`audit_volume`'s arguments from a run's configuration file."""
    from shardtrain_b200.config import load_config

    c = load_config(config_path)
    m = c.model
    model = dict(hidden_size=m.hidden_size, mlp_hidden_size=m.mlp_hidden_size, num_heads=m.num_heads,
                 num_key_value_heads=m.num_key_value_heads or m.num_heads, layers=m.layers,
                 vocab_size=m.vocab_size, seq_len=m.seq_len, tie_word_embeddings=m.tie_word_embeddings)
    return dict(model=model, fsdp=c.parallel.fsdp_degree, tp=c.parallel.tp_degree,
                sp=c.parallel.sp_enabled, local_batch=c.training.local_batch_size)


def audit_benchmark(directory, *, layers: int | None = None, tied: bool | None = None) -> list[str]:
    paths = sorted(Path(directory).glob("benchmark.rank*.json"))
    if not paths:
        return ["no benchmark.rank*.json found"]
    records = {int(p.name.split("rank")[1].split(".")[0]): json.loads(p.read_text()) for p in paths}
    problems: list[str] = []
    for rank, rec in sorted(records.items()):
        def fail(text, rank=rank):
            problems.append(f"rank {rank}: {text}")

        if rec.get("status") != "completed":
            fail(f"status {rec.get('status')!r}")
        if rec.get("oom") or rec.get("errors"):
            fail(f"errors recorded: oom={rec.get('oom')} errors={rec.get('errors')}")
        if rec.get("nonfinite_detected") or rec.get("nonfinite_loss"):
            fail("non-finite loss or gradients recorded")
        steps = rec.get("steps") or []
        if not steps:
            fail("no measured steps")
        if rec.get("overflow_steps"):
            fail(f"{rec['overflow_steps']} overflow steps in the measured region")
        if rec.get("optimizer_updates") != len(steps):
            fail(f"{rec.get('optimizer_updates')} optimizer updates for {len(steps)} steps")
        cfg = rec.get("resolved_config") or rec.get("config") or {}
        resolved = Path(directory) / f"resolved_config.rank{rank}.yaml"
        if not cfg and resolved.exists():
            import yaml

            cfg = yaml.safe_load(resolved.read_text()) or {}
        par, train, model = cfg.get("parallel", {}), cfg.get("training", {}), cfg.get("model", {})
        n_layers = layers if layers is not None else model.get("layers")
        is_tied = tied if tied is not None else model.get("tie_word_embeddings", True)
        own = rec.get("ownership") or {}
        if not own:
            fail("ownership block missing")
        else:
            if own.get("live_buffers") or own.get("live_fullparam_leases"):
                fail(f"live buffers / leases after the run: {own.get('live_buffers')} / "
                     f"{own.get('live_fullparam_leases')}")
            if not own.get("stable_shard_identity"):
                fail("a shard leaf was replaced during the run")
            if not own.get("units_reduced_once_last_microbatch"):
                fail("a unit was not reduced exactly once in the last micro-step")
            if n_layers is not None:
                units = n_layers + 2 + (0 if is_tied else 1)
                leaves = 12 * n_layers + 2 + (0 if is_tied else 1)
                if own.get("unit_count") != units:
                    fail(f"unit_count {own.get('unit_count')}, expected {units}")
                if own.get("persistent_shard_count") != leaves:
                    fail(f"persistent_shard_count {own.get('persistent_shard_count')}, expected {leaves}")
            if own.get("parameter_dtypes") != ["torch.float32"]:
                fail(f"master shards are {own.get('parameter_dtypes')}, expected FP32 only")
            if own.get("gradient_bytes") != own.get("parameter_bytes"):
                fail("gradient bytes differ from parameter bytes")
            if own.get("optimizer_state_parameter_count") not in (0, own.get("persistent_shard_count")):
                fail("optimizer state does not cover every leaf")
        fsdp = par.get("fsdp_degree")
        seq = rec.get("sequence_length") or model.get("seq_len")
        if fsdp and seq and train:
            want = fsdp * train["local_batch_size"] * train["accumulation_steps"] * (seq - 1)
            for row in steps:
                if row.get("valid_tokens") != want:
                    fail(f"step {row.get('step')}: valid_tokens {row.get('valid_tokens')}, expected {want}")
                    break
        for row in steps:
            if row.get("loss") is None or not math.isfinite(row["loss"]):
                fail(f"step {row.get('step')}: loss {row.get('loss')}")
                break
        switches, runtime_cfg = rec.get("runtime_switches") or {}, cfg.get("runtime", {})
        for key, value in switches.items():
            if key in runtime_cfg and runtime_cfg[key] != value:
                fail(f"runtime switch {key}: ran with {value}, configured {runtime_cfg[key]}")
    # across ranks: same step rows, loss within 1e-6
    first = records[min(records)]
    for rank, rec in records.items():
        for a, b in zip(first.get("steps") or [], rec.get("steps") or []):
            same = all(a.get(k) == b.get(k) for k in ("step", "overflow", "loss_scale", "valid_tokens"))
            close = (a.get("loss") is not None and b.get("loss") is not None
                     and abs(a["loss"] - b["loss"]) <= 1e-6 * max(1.0, abs(a["loss"])))
            if not (same and close):
                problems.append(f"rank {rank}: step {a.get('step')} differs from rank {min(records)}")
                break
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    ev = sub.add_parser("events")
    ev.add_argument("directory")
    ev.add_argument("--fsdp", type=int, required=True)
    ev.add_argument("--tp", type=int, default=1)
    ev.add_argument("--layers", type=int, required=True)
    ev.add_argument("--untied", action="store_true")
    ev.add_argument("--policy", default=None, choices=[None, "conservative", "stream_ordered"])
    be = sub.add_parser("benchmark")
    be.add_argument("directory")
    be.add_argument("--layers", type=int, default=None)
    vo = sub.add_parser("volume", help="measured payload of every micro-step against the volume model")
    vo.add_argument("directory")
    vo.add_argument("--config", default=None,
                    help="the run's configuration (default: resolved_config.rank0.yaml in the directory)")
    a = ap.parse_args(argv)
    if a.what == "events":
        problems = audit_event_logs(a.directory, fsdp=a.fsdp, tp=a.tp, layers=a.layers,
                                    tied=not a.untied, policy=a.policy)
    elif a.what == "volume":
        problems = audit_volume(a.directory, **volume_arguments(
            a.config or Path(a.directory) / "resolved_config.rank0.yaml"))
    else:
        problems = audit_benchmark(a.directory, layers=a.layers)
    for line in problems:
        print(line)
    print("accepted" if not problems else f"{len(problems)} violation(s)")
    return 0 if not problems else 1


if __name__ == "__main__":
    raise SystemExit(main())
