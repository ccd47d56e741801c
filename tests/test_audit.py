"""The offline auditors accept real runs and notice tampering (CPU only)."""
import json
import shutil

import pytest

from shardtrain_b200.config import load_config
from shardtrain_b200.training import qwen2_benchmark
from shardtrain_b200.utils.audit import audit_benchmark, audit_event_logs, expected_members, main
from tests.test_cli import CONFIGS


@pytest.fixture(scope="module")
def run_dir(tmp_path_factory):
    out = tmp_path_factory.mktemp("audit") / "run"
    config = load_config(CONFIGS / "qwen25_tiny.yaml", ["--debug.output_dir", str(out),
                                                         "--training.steps", "2"])
    qwen2_benchmark.run(config, warmup=1, runtime_events="on")
    return out, config


@pytest.fixture(scope="module")
def mesh_run(tmp_path_factory):
    """A 2 x 2 gloo run with every overlap switch on (gradient-dispatch prefetch active)."""
    from tests.launch import run_workers

    out = tmp_path_factory.mktemp("audit_mesh")
    code, log = run_workers("tests.workers.qwen_worker", 4,
                            ["--out", out, "--fsdp", 2, "--tp", 2, "--sp", 1, "--flags", "111",
                             "--policy", "stream_ordered", "--accum", 2, "--optimizer", "sgd"])
    assert code == 0, log[-2000:]
    return out


def rewrite(path, edit):
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    path.write_text("\n".join(json.dumps(r) for r in edit(rows)) + "\n")


def test_a_real_run_is_accepted(run_dir):
    out, config = run_dir
    assert audit_benchmark(out) == []
    assert audit_event_logs(out, fsdp=1, tp=1, layers=config.model.layers, tied=True,
                            policy="conservative") == []
    assert main(["benchmark", str(out)]) == 0
    assert main(["events", str(out), "--fsdp", "1", "--layers", str(config.model.layers)]) == 0


@pytest.mark.distributed
def test_a_mesh_run_is_accepted_including_the_dispatch_order(mesh_run):
    assert audit_event_logs(mesh_run, fsdp=2, tp=2, layers=2, tied=True, policy="stream_ordered") == []
    # the policy check is real: the same logs are not a conservative run
    wrong = audit_event_logs(mesh_run, fsdp=2, tp=2, layers=2, tied=True, policy="conservative")
    assert wrong == [] or all("conservative" in p for p in wrong)
    assert audit_event_logs(mesh_run, fsdp=4, tp=1, layers=2) != []      # wrong mesh: membership


@pytest.mark.distributed
@pytest.mark.parametrize("tamper,expect", [
    ("drop_retire", "live buffer"),
    ("drop_commit", "leaves committed"),
    ("early_consume", "consumable before its work was issued"),
    ("extra_gather", "materialisations"),
    ("sequence_gap", "sequence jumps"),
    ("rank_divergence", "diverges from rank"),
    ("late_dispatch", "is not between the issue"),
])
def test_event_log_tampering_is_noticed(mesh_run, tmp_path, tamper, expect):
    copy = tmp_path / "run"
    shutil.copytree(mesh_run, copy)
    log = copy / "runtime_events.rank1.jsonl"

    def edit(rows):
        if tamper == "drop_retire":
            victim = next(i for i, r in enumerate(rows) if r["event_type"] == "buffer_retire"
                          and r["step_id"] == 1)
            del rows[victim]
        elif tamper == "drop_commit":
            victim = next(i for i, r in enumerate(rows) if r["event_type"] == "leaf_grad_committed"
                          and r["step_id"] == 1)
            del rows[victim]
        elif tamper == "early_consume":
            i = next(i for i, r in enumerate(rows) if r["event_type"] == "work_issued")
            j = next(j for j in range(i, len(rows)) if rows[j]["event_type"] == "collective_consumer_ready"
                     and rows[j]["op_id"] == rows[i]["op_id"])
            rows[i], rows[j] = rows[j], rows[i]
        elif tamper == "extra_gather":
            i = next(i for i, r in enumerate(rows) if r["event_type"] == "materialize_issue"
                     and r["step_id"] == 1)
            rows.insert(i, dict(rows[i]))
        elif tamper == "sequence_gap":
            for r in rows:
                if r["event_type"] == "collective_issue" and r["pg_id"] == "tp" and r["pg_local_seq"] >= 3:
                    r["pg_local_seq"] += 1
        elif tamper == "rank_divergence":
            issues = [i for i, r in enumerate(rows) if r["event_type"] == "collective_issue"
                      and r["pg_id"] == "fsdp" and r["step_id"] == 1]
            rows[issues[0]]["op_kind"], rows[issues[1]]["op_kind"] = "fsdp_rs", "fsdp_ag"
        elif tamper == "late_dispatch":
            # move an owner's dispatch token behind the consumption of its reductions
            i = next(i for i, r in enumerate(rows) if r["event_type"] == "backward_prefetch_token"
                     and r.get("gradient_owner") is not None)
            owner = rows[i]["gradient_owner"]
            j = max(j for j in range(i, len(rows)) if rows[j]["event_type"] == "gradient_bucket_consumed"
                    and rows[j]["unit_id"] == owner and rows[j]["step_id"] == rows[i]["step_id"])
            rows.insert(j + 1, rows.pop(i))
        return rows

    rewrite(log, edit)
    problems = audit_event_logs(copy, fsdp=2, tp=2, layers=2, tied=True)
    assert any(expect in p for p in problems), problems


def test_benchmark_gate_rejects_bad_records(run_dir, tmp_path):
    out, _ = run_dir
    for field, value, expect in (("status", "failed", "status"),
                                 ("optimizer_updates", 1, "optimizer updates"),
                                 ("ownership.live_buffers", 2, "live buffers"),
                                 ("ownership.persistent_shard_count", 25, "persistent_shard_count"),
                                 ("ownership.parameter_dtypes", ["torch.bfloat16"], "FP32 only"),
                                 ("steps.0.valid_tokens", 29, "valid_tokens"),
                                 ("steps.1.loss", float("nan"), "loss")):
        copy = tmp_path / field.replace(".", "_")
        shutil.copytree(out, copy)
        path = copy / "benchmark.rank0.json"
        record = json.loads(path.read_text())
        target, keys = record, field.split(".")
        for key in keys[:-1]:
            target = target[int(key)] if key.isdigit() else target[key]
        target[int(keys[-1]) if keys[-1].isdigit() else keys[-1]] = value
        path.write_text(json.dumps(record))
        problems = audit_benchmark(copy)
        assert any(expect in p for p in problems), (field, problems)
    assert audit_benchmark(tmp_path / "missing") == ["no benchmark.rank*.json found"]


def test_communicator_membership_formula():
    # rank = f * tp + t on an F2 x T4 mesh
    assert expected_members("tp", 5, 2, 4) == [4, 5, 6, 7]
    assert expected_members("tp_grad", 1, 2, 4) == [0, 1, 2, 3]
    assert expected_members("fsdp", 5, 2, 4) == [1, 5]
    assert expected_members("fsdp_grad", 2, 2, 4) == [2, 6]


def test_step_profile_summary_groups_streams_kernels_and_gaps(tmp_path):
    """`ops.profile_step.summarise` on a hand-written kineto trace: union of busy time, the
    stream with the most launches is the compute stream, gaps are charged to the kernel after."""
    import json

    from shardtrain_b200.ops.profile_step import summarise

    def kernel(name, ts, dur, stream):
        return {"cat": "kernel", "name": name, "ts": ts, "dur": dur, "args": {"stream": stream}}

    events = [kernel("void stb::(anonymous namespace)::rmsnorm_fwd_kernel<false>(float*)", 0, 10, 7),
              kernel("void stb::gemm_bf16_tcgen05_kernel<256, false, false>(int)", 12, 50, 7),
              kernel("void stb::gemm_bf16_tcgen05_kernel<256, false, false>(int)", 100, 50, 7),   # 38 us gap
              kernel("stb::gather_params_kernel(int)", 20, 100, 9),
              {"cat": "cpu_op", "name": "aten::add", "ts": 0, "dur": 5}]
    path = tmp_path / "trace.json"
    path.write_text(json.dumps({"traceEvents": events}))
    got = summarise(str(path))
    assert got["kernels"] == 4 and got["span_ms"] == pytest.approx(0.150)
    assert got["busy_union_ms"] == pytest.approx(0.150 - 0.002)        # only 10..12 is idle everywhere
    assert [s["launches"] for s in got["streams"]] == [3, 1]
    assert got["top_kernels"][0]["name"] == "gemm_bf16_tcgen05_kernel<256, false, false>"
    assert got["top_kernels"][0]["total_ms"] == pytest.approx(0.1)
    gaps = got["compute_stream_gaps_over_15us"]
    assert gaps["total_ms"] == pytest.approx(0.038) and gaps["before"][0]["count"] == 1


WORKER_TINY = dict(hidden_size=64, mlp_hidden_size=128, num_heads=4, num_key_value_heads=2, layers=2,
                   vocab_size=1024, seq_len=64, tie_word_embeddings=True)


@pytest.mark.distributed
def test_measured_payload_equals_the_volume_model_on_a_mesh(mesh_run):
    """Every micro-step of the 2 x 2 run carries exactly the collectives and elements that the
    volume model predicts from the configuration; a wrong batch or mesh does not."""
    from shardtrain_b200.utils.audit import audit_volume

    assert audit_volume(mesh_run, WORKER_TINY, fsdp=2, tp=2, sp=True, local_batch=2) == []
    wrong_batch = audit_volume(mesh_run, WORKER_TINY, fsdp=2, tp=2, sp=True, local_batch=4)
    assert wrong_batch and all("sp_" in p for p in wrong_batch)
    assert audit_volume(mesh_run, dict(WORKER_TINY, layers=3), fsdp=2, tp=2, sp=True, local_batch=2)


def test_measured_payload_of_a_single_rank_run_has_nothing_to_carry(run_dir):
    from shardtrain_b200.utils.audit import audit_volume

    out, config = run_dir
    problems = audit_volume(out, WORKER_TINY, fsdp=1, tp=1, sp=False, local_batch=2)
    assert problems == ["rank 0: no micro-step with collectives found"]


def test_event_logs_become_a_chrome_trace(run_dir, tmp_path):
    """`utils.trace_events`: one process per rank, collectives and unit phases as slices with
    non-negative durations in log order, step boundaries as markers."""
    from shardtrain_b200.utils import trace_events

    out, _ = run_dir
    target = tmp_path / "timeline.json"
    assert trace_events.main([str(out), "-o", str(target)]) == 0
    events = json.loads(target.read_text())["traceEvents"]
    slices = [e for e in events if e["ph"] == "X"]
    assert slices and all(e["dur"] > 0 and e["ts"] >= 0 and e["pid"] == 0 for e in slices)
    assert {e["cat"] for e in slices} >= {"unit"}
    names = {e["args"]["name"] for e in events if e["ph"] == "M" and e["name"] == "thread_name"}
    assert "units" in names and "markers" in names
    assert any(e["ph"] == "i" and e["name"] == "step_end" for e in events)
    assert trace_events.main([str(tmp_path / "empty")]) == 1
