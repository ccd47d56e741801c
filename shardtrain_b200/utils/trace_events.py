"""Event logs as a timeline: `runtime_events.rank{r}.jsonl` of a run rewritten as one Chrome /
Perfetto trace (`chrome://tracing`, ui.perfetto.dev), without any profiler having been attached.

    python -m shardtrain_b200.utils.trace_events runs/<dir> -o timeline.json

One process per rank.  Every collective becomes a slice on the track of the stream it was issued
on, from its `collective_issue` to its `collective_consumer_ready` (host clock: the time a
consumer could first take the result, not the device's execution time); a unit's life in a
micro-step (`unit_forward` .. `fullparams_retired` / `unit_pre_backward` .. `unit_grads_ready`)
becomes slices on a `units` track; step boundaries, prefetch decisions and dependency edges of
kind PG_ORDER become instant markers.  The log's own fields travel in `args`.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from shardtrain_b200.utils.audit import read_events

INSTANTS = {"step_end", "optimizer_ready", "prefetch_boundary", "parameter_shards_ready",
            "backward_prefetch_token", "runtime_failed"}
KEEP = ("step_id", "unit_id", "phase", "kind", "numel", "dtype", "pg_id", "pg_local_seq", "group_role",
        "group_members", "dependency_type", "target_unit", "scheduling_boundary", "reason")


def _args(row: dict) -> dict:
    return {k: row[k] for k in KEEP if row.get(k) is not None}


def to_trace(logs: dict[int, list[dict]]) -> dict:
    origin = min((r["CPU_timestamp"] for rows in logs.values() for r in rows if "CPU_timestamp" in r),
                 default=0.0)
    micro = lambda row: (row["CPU_timestamp"] - origin) * 1e6          # noqa: E731
    events, tracks = [], {}

    def track(rank, name):
        key = (rank, name)
        if key not in tracks:
            tracks[key] = len([k for k in tracks if k[0] == rank]) + 1
            events.append({"ph": "M", "name": "thread_name", "pid": rank, "tid": tracks[key],
                           "args": {"name": name}})
        return tracks[key]

    for rank, rows in sorted(logs.items()):
        events.append({"ph": "M", "name": "process_name", "pid": rank, "args": {"name": f"rank {rank}"}})
        issued, open_units = {}, {}
        for row in rows:
            if "CPU_timestamp" not in row:
                continue
            kind, now = row["event_type"], micro(row)
            if kind == "collective_issue":
                issued[row["op_id"]] = row
            elif kind == "collective_consumer_ready" and row.get("op_id") in issued:
                first = issued.pop(row["op_id"])
                events.append({"ph": "X", "name": first.get("kind") or "collective", "pid": rank,
                               "tid": track(rank, f"stream {first.get('issue_stream') or 'cpu'}"),
                               "ts": micro(first), "dur": max(now - micro(first), 0.01),
                               "cat": "collective", "args": _args(first)})
            elif kind in ("unit_forward", "unit_pre_backward"):
                open_units[(row.get("unit_id"), row.get("phase"))] = row
            elif kind in ("fullparams_retired", "unit_grads_ready", "FWD_RETAINED", "RESHARDED"):
                for key in [k for k in open_units if k[0] == row.get("unit_id")]:
                    first = open_units.pop(key)
                    events.append({"ph": "X", "name": f"U{key[0]} {key[1]}", "pid": rank,
                                   "tid": track(rank, "units"), "ts": micro(first),
                                   "dur": max(now - micro(first), 0.01), "cat": "unit",
                                   "args": _args(first)})
            elif kind in INSTANTS or (kind == "dependency_edge" and row.get("dependency_type") == "PG_ORDER"):
                events.append({"ph": "i", "s": "t", "name": kind, "pid": rank,
                               "tid": track(rank, "markers"), "ts": now, "args": _args(row)})
    return {"traceEvents": events, "displayTimeUnit": "ms"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory")
    ap.add_argument("-o", "--output", default=None, help="default: <directory>/timeline.json")
    a = ap.parse_args(argv)
    logs = read_events(a.directory)
    if not logs:
        print(f"no runtime_events.rank*.jsonl in {a.directory}")
        return 1
    trace = to_trace(logs)
    out = Path(a.output or Path(a.directory) / "timeline.json")
    out.write_text(json.dumps(trace))
    slices = sum(e["ph"] == "X" for e in trace["traceEvents"])
    print(f"{out}: {len(logs)} rank(s), {slices} slices, {len(trace['traceEvents'])} events")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
