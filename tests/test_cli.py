"""Entry points: `shardtrain_b200.train` routing and the Qwen benchmark's records
(modelled on tests/test_train_cli.py and tests/test_qwen2_benchmark.py of the reference)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from shardtrain_b200 import train
from shardtrain_b200.config import ConfigError, load_config
from shardtrain_b200.training import qwen2_benchmark
from tests.launch import ROOT, run_workers

CONFIGS = ROOT / "configs"


def test_every_preset_parses():
    names = sorted(p.name for p in CONFIGS.glob("*.yaml") if not p.name.endswith("_config.yaml"))
    assert {"qwen25_tiny.yaml", "qwen25_1p5b_b200.yaml", "correctness.yaml", "tp_sp.yaml",
            "runtime_cpu.yaml", "smoke_gloo.yaml"} <= set(names)
    for name in names:
        load_config(CONFIGS / name)
    for name, strategy in (("S-F", "F4T1"), ("S-H", "F2T2/SP"), ("N-F", "F4T1"), ("N-H", "F2T2/SP")):
        preset = load_config(CONFIGS / "fsdp4_hybrid_2x2" / f"{name}.yaml")
        assert preset.parallel.strategy == strategy
        assert preset.training.local_batch_size * preset.parallel.fsdp_degree == 8
    headline = load_config(CONFIGS / "qwen25_1p5b_b200.yaml")
    assert headline.parallel.strategy == "F8T1"
    assert headline.training.local_batch_size * headline.parallel.fsdp_degree == 8
    large = load_config(CONFIGS / "qwen25_7b_b200.yaml")
    large.validate(8, mode="runtime")
    assert large.parallel.strategy == "F2T4/SP" and not large.model.tie_word_embeddings
    assert large.training.local_batch_size * large.parallel.fsdp_degree * 2 == 16   # global batch


def test_train_toy_reference_writes_step_rows(tmp_path):
    out = tmp_path / "run"
    assert train.main(["--config", str(CONFIGS / "correctness.yaml"), "--debug.output_dir", str(out),
                       "--training.steps", "2"]) == 0
    rows = json.loads((out / "steps.rank0.json").read_text())
    assert [r["step"] for r in rows] == [0, 1]
    assert rows[1]["loss"] != rows[0]["loss"]
    assert (out / "environment.rank0.json").exists() and (out / "resolved_config.rank0.yaml").exists()


def test_train_toy_through_runtime_flag(tmp_path):
    out = tmp_path / "run"
    assert train.main(["--config", str(CONFIGS / "correctness.yaml"), "--sharded-runtime",
                       "--debug.output_dir", str(out), "--training.steps", "2"]) == 0
    assert len(json.loads((out / "steps.rank0.json").read_text())) == 2
    assert (out / "runtime_events.rank0.jsonl").exists()


def test_train_qwen_routes_to_benchmark(tmp_path):
    out = tmp_path / "run"
    assert train.main(["--config", str(CONFIGS / "qwen25_tiny.yaml"), "--debug.output_dir", str(out),
                       "--training.steps", "2"]) == 0
    record = json.loads((out / "benchmark.rank0.json").read_text())
    assert record["status"] == "completed" and record["warmup"] == 0
    assert record["steady_steps_completed"] == 2


def test_bad_override_is_a_usage_error(tmp_path, capsys):
    with pytest.raises(SystemExit) as info:
        train.main(["--config", str(CONFIGS / "correctness.yaml"), "--training.nonsense", "1"])
    assert info.value.code == 2
    assert "nonsense" in capsys.readouterr().err


def test_benchmark_record_contents_and_directory_reuse(tmp_path):
    out = tmp_path / "bench"
    config = load_config(CONFIGS / "qwen25_tiny.yaml", ["--debug.output_dir", str(out),
                                                         "--training.steps", "3"])
    record = qwen2_benchmark.run(config, warmup=1, peak_tflops_per_gpu=100.0)
    assert record["status"] == "completed" and len(record["warmup_steps"]) == 1
    assert [row["measured_step"] for row in record["steps"]] == [0, 1, 2]
    assert record["step_seconds_p50"] <= record["step_seconds_p95"]
    assert record["global_batch"] == 2 and record["steps"][0]["valid_tokens"] == 2 * 15
    own = record["ownership"]
    assert own["stable_shard_identity"] and own["units_reduced_once_last_microbatch"]
    assert own["live_buffers"] == 0 and own["live_fullparam_leases"] == 0
    assert own["optimizer_tensor_bytes"] == 2 * own["parameter_bytes"]
    perf = record["performance"]
    assert perf["mfu_percent"] > 0 and perf["unprofiled_timing"]
    assert record["model_source"]["tied_aliases"] == {"lm_head.weight": "model.embed_tokens.weight"}
    assert json.loads((out / "benchmark.rank0.json").read_text())["input_batch_digest"] == \
        record["input_batch_digest"]
    with pytest.raises(ConfigError, match="already contains rank 0"):
        qwen2_benchmark.run(config, warmup=0)


def test_benchmark_rejects_bad_arguments(tmp_path):
    config = load_config(CONFIGS / "qwen25_tiny.yaml", ["--debug.output_dir", str(tmp_path / "x")])
    for kwargs in ({"warmup": -1}, {"profile_mode": "nsight"}, {"profile_mode": "bogus"},
                   {"profile_detail": "bogus"}, {"peak_tflops_per_gpu": 0.0}):
        with pytest.raises(ConfigError):
            qwen2_benchmark.run(config, **kwargs)
    toy = load_config(CONFIGS / "correctness.yaml")
    with pytest.raises(ConfigError, match="qwen2"):
        qwen2_benchmark.run(toy)


def test_benchmark_failure_is_recorded_then_raised(tmp_path, monkeypatch):
    out = tmp_path / "bench"
    config = load_config(CONFIGS / "qwen25_tiny.yaml", ["--debug.output_dir", str(out)])

    def explode(self, *a, **k):
        raise RuntimeError("CUDA out of memory (injected on the host)")

    monkeypatch.setattr(qwen2_benchmark.QwenTrainer, "train_step", explode)
    with pytest.raises(RuntimeError, match="injected"):
        qwen2_benchmark.run(config, warmup=0)
    record = json.loads((out / "benchmark.rank0.json").read_text())
    assert record["status"] == "failed" and record["oom"] and record["steady_steps_completed"] == 0


def test_benchmark_torch_profile_mode_on_cpu(tmp_path):
    out = tmp_path / "bench"
    config = load_config(CONFIGS / "qwen25_tiny.yaml", ["--debug.output_dir", str(out),
                                                         "--training.steps", "1"])
    record = qwen2_benchmark.run(config, warmup=0, profile_mode="torch")
    assert record["runtime_events_enabled"] and not record["performance"]["unprofiled_timing"]
    assert (out / "profile.rank0.json").exists() and (out / "profiling.rank0.json").exists()
    assert (out / "runtime_events.rank0.jsonl").exists()


def test_percentile_interpolates():
    assert qwen2_benchmark.percentile([], 0.5) is None
    assert qwen2_benchmark.percentile([4.0], 0.95) == 4.0
    assert qwen2_benchmark.percentile([1.0, 2.0, 3.0, 4.0], 0.5) == 2.5


def test_module_entry_point_runs_as_a_script(tmp_path):
    done = subprocess.run([sys.executable, "-m", "shardtrain_b200.train", "--help"], cwd=ROOT,
                          capture_output=True, text=True, timeout=120)
    assert done.returncode == 0 and "--smoke-groups" in done.stdout


@pytest.mark.distributed
def test_smoke_groups_on_four_gloo_ranks(tmp_path):
    out = tmp_path / "smoke"
    code, log = run_workers("shardtrain_b200.train", 4,
                            ["--config", CONFIGS / "smoke_gloo.yaml", "--smoke-groups",
                             "--debug.output_dir", out])
    assert code == 0, log[-3000:]
    for rank in range(4):
        result = json.loads((out / f"smoke.rank{rank}.json").read_text())
        assert set(result) >= {"tp", "fsdp"}
    assert not list(Path(out).glob("steps.rank*.json"))


@pytest.mark.distributed
def test_qwen_benchmark_two_ranks_fsdp(tmp_path):
    out = tmp_path / "bench"
    code, log = run_workers("shardtrain_b200.training.qwen2_benchmark", 2,
                            ["--config", CONFIGS / "qwen25_tiny.yaml", "--warmup", "1",
                             "--parallel.fsdp_degree", "2", "--training.steps", "2",
                             "--runtime.forward_prefetch", "true", "--runtime.backward_prefetch",
                             "true", "--runtime.async_grad_rs", "true", "--debug.output_dir", out])
    assert code == 0, log[-3000:]
    records = [json.loads((out / f"benchmark.rank{r}.json").read_text()) for r in range(2)]
    assert all(r["status"] == "completed" and r["global_batch"] == 4 for r in records)
    assert records[0]["steps"][0]["max_rank_seconds"] == records[1]["steps"][0]["max_rank_seconds"]
    assert records[0]["steps"][1]["loss"] == pytest.approx(records[1]["steps"][1]["loss"])


def test_native_fsdp2_baseline_matches_the_sharded_runtime_single_rank(tmp_path):
    """Same model, same name-stable initialisation, same batch: the PyTorch-native engine and
    this package's runtime report the same losses step by step."""
    from shardtrain_b200.training import qwen2_native_baseline

    overrides = ["--training.steps", "3"]
    ours = qwen2_benchmark.run(load_config(
        CONFIGS / "qwen25_tiny.yaml", overrides + ["--debug.output_dir", str(tmp_path / "ours")]))
    native = qwen2_native_baseline.run(load_config(
        CONFIGS / "qwen25_tiny.yaml", overrides + ["--debug.output_dir", str(tmp_path / "native")]))
    assert native["engine"] == "native_fsdp2" and native["status"] == "completed"
    for a, b in zip(ours["steps"], native["steps"]):
        assert a["loss"] == pytest.approx(b["loss"], rel=1e-5)
        assert a["valid_tokens"] == b["valid_tokens"]
    assert native["performance"]["model_unique_parameters"] == \
        ours["performance"]["model_unique_parameters"]
    with pytest.raises(ConfigError, match="WORLD_SIZE=1 does not match"):
        qwen2_native_baseline.run(load_config(
            CONFIGS / "qwen25_tiny.yaml", ["--parallel.tp_degree", "2", "--parallel.sp_enabled", "true",
                                           "--debug.output_dir", str(tmp_path / "refused")]))


@pytest.mark.distributed
def test_native_fsdp2_baseline_two_ranks_matches_runtime(tmp_path):
    common = ["--config", CONFIGS / "qwen25_tiny.yaml", "--warmup", "0", "--parallel.fsdp_degree", "2",
              "--training.steps", "2", "--runtime.forward_prefetch", "true",
              "--runtime.backward_prefetch", "true"]
    losses = {}
    for module in ("qwen2_native_baseline", "qwen2_benchmark"):
        out = tmp_path / module
        code, log = run_workers(f"shardtrain_b200.training.{module}", 2, common + ["--debug.output_dir", out])
        assert code == 0, log[-3000:]
        record = json.loads((out / "benchmark.rank0.json").read_text())
        assert record["status"] == "completed"
        losses[module] = [row["loss"] for row in record["steps"]]
    assert losses["qwen2_native_baseline"] == pytest.approx(losses["qwen2_benchmark"], rel=1e-5)


def test_compare_engines_reads_two_runs_and_refuses_different_workloads(tmp_path, capsys):
    from shardtrain_b200.training import qwen2_native_baseline
    from shardtrain_b200.utils import compare_engines

    base = ["--training.steps", "2"]
    qwen2_benchmark.run(load_config(CONFIGS / "qwen25_tiny.yaml", base + ["--debug.output_dir", str(tmp_path / "a")]))
    qwen2_native_baseline.run(load_config(CONFIGS / "qwen25_tiny.yaml", base + ["--debug.output_dir", str(tmp_path / "b")]))
    qwen2_benchmark.run(load_config(CONFIGS / "qwen25_tiny.yaml",
                                    base + ["--training.local_batch_size", "4", "--debug.output_dir", str(tmp_path / "c")]))
    result = compare_engines.compare(compare_engines.load_run(tmp_path / "a"), compare_engines.load_run(tmp_path / "b"))
    assert result["a"]["engine"] == "shardtrain_b200" and result["b"]["engine"] == "native_fsdp2"
    assert abs(result["first_loss_difference"]) < 1e-4 and result["throughput_ratio_a_over_b"] > 0
    assert compare_engines.main([str(tmp_path / "a"), str(tmp_path / "b")]) == 0
    assert "a / b throughput" in capsys.readouterr().out
    with pytest.raises(ValueError, match="different workloads"):
        compare_engines.compare(compare_engines.load_run(tmp_path / "a"), compare_engines.load_run(tmp_path / "c"))
    with pytest.raises(FileNotFoundError):
        compare_engines.load_run(tmp_path / "missing")


@pytest.mark.distributed
def test_native_baseline_fsdp_x_tp_mesh_matches_runtime(tmp_path):
    """F2 x T2 without SP on 4 gloo ranks: DTensor Colwise / Rowwise plan + fully_shard against
    this package's runtime on the same mesh."""
    common = ["--config", CONFIGS / "qwen25_tiny.yaml", "--warmup", "0", "--parallel.fsdp_degree", "2",
              "--parallel.tp_degree", "2", "--training.steps", "2"]
    losses = {}
    for module in ("qwen2_native_baseline", "qwen2_benchmark"):
        out = tmp_path / module
        code, log = run_workers(f"shardtrain_b200.training.{module}", 4, common + ["--debug.output_dir", out])
        assert code == 0, log[-3000:]
        records = [json.loads((out / f"benchmark.rank{r}.json").read_text()) for r in range(4)]
        assert all(r["status"] == "completed" for r in records)
        losses[module] = [row["loss"] for row in records[0]["steps"]]
    assert losses["qwen2_native_baseline"] == pytest.approx(losses["qwen2_benchmark"], rel=1e-5)


@pytest.mark.distributed
def test_native_baseline_sequence_parallel_mesh_matches_runtime(tmp_path):
    """F2 x T2 with sequence parallelism on 4 gloo ranks: DTensor SequenceParallel norms, one
    gathered input per block, row-parallel outputs scattered back to the sequence shard --
    against this package's runtime on the same mesh, same weights, same batches."""
    common = ["--config", CONFIGS / "qwen25_tiny.yaml", "--warmup", "0", "--parallel.fsdp_degree", "2",
              "--parallel.tp_degree", "2", "--parallel.sp_enabled", "true", "--training.steps", "3",
              "--training.accumulation_steps", "2", "--training.local_batch_size", "2"]
    losses = {}
    for module in ("qwen2_native_baseline", "qwen2_benchmark"):
        out = tmp_path / module
        code, log = run_workers(f"shardtrain_b200.training.{module}", 4, common + ["--debug.output_dir", out])
        assert code == 0, log[-3000:]
        records = [json.loads((out / f"benchmark.rank{r}.json").read_text()) for r in range(4)]
        assert all(r["status"] == "completed" for r in records)
        assert len({tuple(row["loss"] for row in r["steps"]) for r in records}) == 1   # all ranks agree
        losses[module] = [row["loss"] for row in records[0]["steps"]]
        if module == "qwen2_native_baseline":
            assert records[0]["sharding"]["sequence_parallel"] is True
    # three optimizer steps: the engines stay together only if the TP-replicated parameters
    # (embedding, norms) received the gradient summed over the sequence shards
    assert losses["qwen2_native_baseline"] == pytest.approx(losses["qwen2_benchmark"], rel=2e-5)
    assert losses["qwen2_benchmark"][2] < losses["qwen2_benchmark"][0]


def test_native_trainer_loss_scale_backs_off_and_skips_on_overflow():
    """The native engine's hand-kept fp16 loss scale: an overflow skips the update and halves the
    scale, clean steps leave it alone until the growth interval doubles it (CPU: the dtype is
    forced after construction, only the bookkeeping is exercised)."""
    import torch

    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.training.qwen2_native_baseline import NativeQwenTrainer

    torch.manual_seed(0)
    model = Qwen2CausalLM(Qwen2ModelConfig(vocab_size=64, hidden_size=32, intermediate_size=64,
                                           num_hidden_layers=1, num_attention_heads=4,
                                           num_key_value_heads=2))
    trainer = NativeQwenTrainer(model, 1e-3, dtype="fp32", optimizer="adamw", accumulation_steps=1,
                                device=torch.device("cpu"), group=None)
    trainer.dynamic_scale, trainer.loss_scale, trainer.growth_interval = True, 128.0, 2
    ids = torch.randint(0, 64, (2, 8))
    before = [p.detach().clone() for p in model.parameters()]
    hook = model.lm_head.weight.register_hook(lambda g: torch.full_like(g, float("inf")))
    skipped = trainer.train_step(ids, ids)
    hook.remove()
    assert skipped.overflow and trainer.loss_scale == 64.0
    assert all(torch.equal(a, b) for a, b in zip(before, model.parameters()))
    first = trainer.train_step(ids, ids)
    assert not first.overflow and trainer.loss_scale == 64.0
    assert not all(torch.equal(a, b) for a, b in zip(before, model.parameters()))
    trainer.train_step(ids, ids)
    assert trainer.loss_scale == 128.0            # two clean steps: the scale grew back
