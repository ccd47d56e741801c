"""Multi-process CPU/gloo runs of the tiny Qwen2 through torchrun on localhost."""
import json

import pytest

from tests.launch import run_workers

pytestmark = pytest.mark.distributed

CASES = [
    # name, nproc, worker arguments
    ("f2t1", 2, ["--fsdp", 2, "--optimizer", "sgd"]),
    ("f2t1_adamw_accum", 2, ["--fsdp", 2, "--optimizer", "adamw", "--accum", 2]),
    ("f1t2_sp", 2, ["--tp", 2, "--sp", 1, "--optimizer", "sgd"]),
    ("f1t2_nosp", 2, ["--tp", 2, "--sp", 0, "--optimizer", "sgd"]),
    ("f2t2_sp_dispatch", 4, ["--fsdp", 2, "--tp", 2, "--sp", 1, "--flags", "111", "--policy",
                             "stream_ordered", "--accum", 2, "--optimizer", "sgd"]),
    ("f4t1_untied", 4, ["--fsdp", 4, "--flags", "110", "--policy", "stream_ordered", "--tied", 0,
                        "--optimizer", "sgd"]),
    # the 8-rank meshes of the reference's gloo gate (tests/distributed/test_runtime.py:110-129)
    ("f4t2_sp", 8, ["--fsdp", 4, "--tp", 2, "--sp", 1, "--flags", "111", "--policy", "stream_ordered",
                    "--optimizer", "sgd"]),
    ("f2t4_sp", 8, ["--fsdp", 2, "--tp", 4, "--sp", 1, "--flags", "111", "--policy", "stream_ordered",
                    "--optimizer", "sgd", "--shape", "tiny4", "--tied", 0]),
    ("f8t1", 8, ["--fsdp", 8, "--flags", "111", "--policy", "stream_ordered", "--optimizer", "sgd"]),
]


def degree(args, flag):
    return int(args[args.index(flag) + 1]) if flag in args else 1


def assert_same_sequence_per_communicator(results, fsdp, tp):
    """Every member of a communicator issued the same collectives in the same order (kind, unit,
    phase): the invariant that keeps blocking collectives from pairing up wrongly.  Rank r sits
    at (f, t) = divmod(r, tp); tp / tp_grad communicators fix f, fsdp / fsdp_grad fix t."""
    def issued(rank, role):
        return [tuple(entry[1:]) for entry in results[rank]["seq"] if entry[0] == role]

    groups = []
    for role in ("tp", "tp_grad"):
        groups += [(role, [f * tp + t for t in range(tp)]) for f in range(fsdp)]
    for role in ("fsdp", "fsdp_grad"):
        groups += [(role, [f * tp + t for f in range(fsdp)]) for t in range(tp)]
    checked = 0
    for role, members in groups:
        sequences = [issued(m, role) for m in members]
        for member, sequence in zip(members[1:], sequences[1:]):
            assert sequence == sequences[0], (
                f"{role} communicator {members}: rank {member} diverges from rank {members[0]}")
        checked += len(sequences[0]) * (len(members) > 1)
    assert checked > 0, "no multi-member communicator issued anything"


def load(out, ranks):
    return [json.loads((out / f"result.rank{r}.json").read_text()) for r in range(ranks)]


@pytest.mark.parametrize("name,nproc,args", CASES, ids=[c[0] for c in CASES])
def test_sharded_training_matches_dense(tmp_path, name, nproc, args):
    code, log = run_workers("tests.workers.qwen_worker", nproc, ["--out", tmp_path, *args],
                            timeout=240 if nproc < 8 else 420)
    assert code == 0, log[-3000:]
    results = load(tmp_path, nproc)
    adamw = "adamw" in [str(a) for a in args]
    for r in results:
        for row in r["rows"]:
            assert row["loss"] == pytest.approx(row["ref"], rel=3e-6)
        # AdamW normalises the update, so near-cancelling gradients move parameters by up to
        # ~lr whatever the summation order; SGD runs must agree tightly
        assert r["param_err"] < (2e-4 if adamw else 5e-6)
        assert r["shard_ok"] and r["live"] == 0
    assert_same_sequence_per_communicator(results, degree(args, "--fsdp"), degree(args, "--tp"))
    # the offline auditor accepts the run's event logs (buffer lifetimes, collective order,
    # per-step counts, policy edges, gradient-dispatch order, cross-rank sequences)
    from shardtrain_b200.utils.audit import audit_event_logs

    policy = args[args.index("--policy") + 1] if "--policy" in args else "conservative"
    tied_model = not ("--tied" in args)
    assert audit_event_logs(tmp_path, fsdp=degree(args, "--fsdp"), tp=degree(args, "--tp"), layers=2,
                            tied=tied_model, policy=policy) == []
    first = results[0]
    layers, steps = 2, 3
    micro = 2 if "--accum" in args else 1
    tied = not ("--tied" in args)
    if "--fsdp" in args:
        per_micro = 2 * layers + 2 if tied else 2 * layers + 5
        assert first["kinds"]["fsdp_ag"] == steps * micro * per_micro
    if "--sp" in args and args[args.index("--sp") + 1] == 1:
        assert first["kinds"]["sp_ag"] == steps * micro * 6 * layers
        assert first["kinds"]["sp_rs_math_allreduce"] == steps * micro * 4 * layers
    assert first["names"][0] == "model.embed_tokens.weight"


def test_initialisation_mismatch_is_rejected_on_every_rank(tmp_path):
    code, log = run_workers("tests.workers.qwen_worker", 2, ["--out", tmp_path, "--fsdp", 2, "--mismatch", 1])
    assert code != 0
    assert "differs across ranks" in log
    assert not list(tmp_path.glob("result.rank*.json"))


def test_wrong_world_size_fails_fast(tmp_path):
    code, log = run_workers("tests.workers.qwen_worker", 2, ["--out", tmp_path, "--fsdp", 4], timeout=120)
    assert code != 0
    assert "world size" in log.lower()


def test_nonfinite_gradient_on_one_rank_fails_every_rank_in_the_same_step(tmp_path):
    """Host-side fault injection: rank 1 poisons one shard gradient in step 1.  The finite vote
    makes every rank raise in that step, the runtime is FAILED everywhere and refuses the next
    step instead of continuing with diverged collective order."""
    import json

    code, log = run_workers("tests.workers.qwen_worker", 2,
                            ["--out", tmp_path, "--fsdp", 2, "--optimizer", "sgd",
                             "--inject-inf-rank", 1])
    assert code == 0, log[-3000:]
    for rank in range(2):
        record = json.loads((tmp_path / f"failure.rank{rank}.json").read_text())
        assert record["step"] == 1 and "Nonfinite" in record["error"]
        assert record["failed"] and record["refused_again"]
    assert not list(tmp_path.glob("result.rank*.json"))


def test_rank_skew_does_not_change_results(tmp_path):
    """One rank is 50 ms late (host sleep) before every step, with every overlap switch on: the
    consumer-ordered waits absorb the skew and training still matches the dense model."""
    import json

    code, log = run_workers("tests.workers.qwen_worker", 2,
                            ["--out", tmp_path, "--fsdp", 2, "--optimizer", "sgd", "--flags", "111",
                             "--delay-rank", 0])
    assert code == 0, log[-3000:]
    for rank in range(2):
        record = json.loads((tmp_path / f"result.rank{rank}.json").read_text())
        assert record["param_err"] < 1e-5
        assert all(abs(row["loss"] - row["ref"]) < 1e-4 for row in record["rows"])


@pytest.mark.parametrize("sp", [0, 1], ids=["tp", "tp_sp"])
def test_legacy_synchronous_tp_path_follows_the_dense_model(tmp_path, sp):
    """The blocking TP / TP+SP conversion of the toy stack (column / row linears over the
    conjugate collective maps, shared sequence gather, replicated-gradient SUM) on 2 gloo ranks:
    losses and reassembled parameters track the unsharded trainer for three SGD steps."""
    code, log = run_workers("tests.workers.tp_sp_worker", 2, ["--out", tmp_path, "--sp", sp])
    assert code == 0, log[-3000:]
    for rank in range(2):
        record = json.loads((tmp_path / f"tp.rank{rank}.json").read_text())
        for row in record["rows"]:
            assert row["loss"] == pytest.approx(row["ref"], rel=2e-6)
        assert record["worst"] < 2e-6
        assert record["column_dim"] == 0 and record["heads"] == 2 and record["local_rows"] == 16
