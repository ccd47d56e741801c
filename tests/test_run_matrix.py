"""The staged acceptance runner: planning is pure, a dry run writes the plan and launches nothing,
a real stage passes its gates on CPU, and a run that exceeds its limit is reported, not waited for."""
import json
import sys

from shardtrain_b200.utils import run_matrix


def test_plan_covers_the_meshes_that_fit_and_all_flag_triples():
    cases = run_matrix.plan_cases(("groups", "flags", "meshes", "policies"), max_ranks=4)
    by_stage = {}
    for case in cases:
        by_stage.setdefault(case.stage, []).append(case)
    assert [(c.fsdp, c.tp) for c in by_stage["groups"]] == [(1, 1), (2, 1), (1, 2), (2, 2), (4, 1)]
    assert len({c.flags for c in by_stage["flags"]}) == 8
    assert {(c.fsdp, c.tp) for c in by_stage["flags"]} == {(2, 2)}
    assert {c.policy for c in by_stage["policies"]} == {"conservative", "stream_ordered"}
    assert len({c.name for c in cases}) == len(cases)
    eight = run_matrix.plan_cases(("meshes",), max_ranks=8)
    assert {(c.fsdp, c.tp) for c in eight} >= {(4, 2), (2, 4), (8, 1)}
    assert run_matrix.largest_hybrid(8) == (4, 2) and run_matrix.largest_hybrid(1) == (1, 1)


def test_dry_run_writes_the_plan_and_every_case_directory(tmp_path):
    out = tmp_path / "matrix"
    assert run_matrix.main(["--stages", "groups,flags", "--max-ranks", "2", "--dry-run",
                            "--output", str(out)]) == 0
    plan = json.loads((out / "plan.json").read_text())
    assert len(plan) == 3 + 8 and not (out / "summary.json").exists()
    for row in plan:
        command = json.loads(open(f"{row['directory']}/launch_command.json").read())
        assert command[:3] == [sys.executable, "-m", "torch.distributed.run"]
        assert "127.0.0.1" in " ".join(command)


def test_policy_stage_runs_on_cpu_and_passes_the_audits(tmp_path):
    out = tmp_path / "matrix"
    assert run_matrix.main(["--stages", "groups,policies", "--max-ranks", "2", "--output", str(out),
                            "--limit", "240"]) == 0
    summary = json.loads((out / "summary.json").read_text())
    assert len(summary) == 3 + 2 and all(row["passed"] for row in summary)


def test_a_run_over_its_limit_is_killed_and_reported(tmp_path):
    case = run_matrix.Case("groups", 1, 1, (False,) * 3, "conservative", "smoke")
    case.directory = str(tmp_path)
    case.command = [sys.executable, "-c", "import time; time.sleep(60)"]
    status, seconds = run_matrix.launch(case, limit=1.0)
    assert status < 0 and seconds < 30
    assert run_matrix.gate(case, status, 2, True) == [f"launcher exit status {status}"]
