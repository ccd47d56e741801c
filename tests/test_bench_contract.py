"""Host-side pieces of the benchmark harness (`bench.py`): defaults, strategy parsing, the
configuration it builds per GPU count, the second-session rendezvous, the reference arm's
`unavailable` line.  Nothing here needs a GPU."""
import json
import sys
from types import SimpleNamespace

import pytest

import bench


def args_for(**changes):
    base = dict(gpus=1, steps=10, warmup=3, model="1.5b", strategy="", layers=0, global_batch=16,
                retain=0, backend="auto", fp32_wire=False, fused_allgather="auto", seq_pull=False,
                nvls="off", no_graphs=False, no_secondary=False)
    base.update(changes)
    return SimpleNamespace(**base)


def test_defaults_are_one_gpu_and_a_run_of_minutes(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert (args.gpus, args.impl, args.model, args.strategy) == (1, "ours", "1.5b", "")
    assert args.warmup >= 3 and 1 <= args.steps <= 30
    assert (args.nvls, args.fused_allgather, args.seq_pull, args.no_graphs) == ("off", "auto", False, False)


def test_strategy_names_and_the_hybrid_of_each_gpu_count():
    assert bench.resolve_strategy(args_for(gpus=8)) == (8, 1, False)
    assert bench.resolve_strategy(args_for(gpus=8, strategy="F4T2/SP")) == (4, 2, True)
    assert bench.resolve_strategy(args_for(gpus=8, strategy="f2t4/sp")) == (2, 4, True)
    assert bench.resolve_strategy(args_for(gpus=2, strategy="F1T2")) == (1, 2, False)
    assert bench.HYBRID == {2: (1, 2, True), 4: (2, 2, True), 8: (4, 2, True)}
    for gpus, (f, t, _) in bench.HYBRID.items():
        assert f * t == gpus


@pytest.mark.parametrize("gpus,fsdp,tp,sp,local", [(1, 1, 1, False, 8), (2, 2, 1, False, 4),
                                                    (4, 4, 1, False, 2), (8, 8, 1, False, 1),
                                                    (8, 4, 2, True, 2), (4, 2, 2, True, 4)])
def test_the_workload_is_the_named_one_at_every_gpu_count(gpus, fsdp, tp, sp, local):
    cfg = bench.qwen15b_dict(args_for(gpus=gpus), fsdp, tp, sp)
    model, training, runtime = cfg["model"], cfg["training"], cfg["runtime"]
    assert (model["layers"], model["hidden_size"], model["vocab_size"], model["seq_len"]) == (28, 1536, 151936, 512)
    assert (training["dtype"], training["optimizer"], training["accumulation_steps"]) == ("bf16", "adamw", 2)
    # global batch 16 = FSDP degree x micro-steps x local batch: strong scaling
    assert training["local_batch_size"] == local and fsdp * 2 * local == 16
    assert all(runtime[k] for k in ("reshard_after_forward", "forward_prefetch", "backward_prefetch", "async_grad_rs"))
    assert runtime["communication_policy"] == "stream_ordered"
    assert bench.valid_labels(args_for()) == 16 * 511 == bench.VALID_LABELS_PER_STEP
    assert bench.valid_labels(args_for(model="7b")) == 16 * 2047
    bench.qwen15b_config(args_for(gpus=gpus), fsdp, tp, sp)       # validates as a configuration


def test_second_session_moves_to_its_own_store(monkeypatch):
    monkeypatch.setenv("MASTER_PORT", "29500")
    monkeypatch.setenv("TORCHELASTIC_USE_AGENT_STORE", "True")
    bench.next_rendezvous()
    import os

    assert os.environ["MASTER_PORT"] == "29501" and os.environ["TORCHELASTIC_USE_AGENT_STORE"] == "False"
    monkeypatch.delenv("MASTER_PORT")
    bench.next_rendezvous()                                       # single process: nothing to move
    assert "MASTER_PORT" not in os.environ


def test_reference_arm_reports_unavailable_when_the_package_is_missing(monkeypatch, tmp_path, capsys):
    from baseline import reference_arm

    monkeypatch.setattr(reference_arm, "REF", tmp_path / "nothing_here")
    monkeypatch.delenv("RANK", raising=False)
    reference_arm.run_reference(args_for(impl="reference"))
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "not installed" in line["unavailable"]
