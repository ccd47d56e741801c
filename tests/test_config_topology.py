import pytest
import yaml

from shardtrain_b200.config import (Config, ConfigError, config_from_dict, load_config,
                                    parse_strategy, with_strategy)
from shardtrain_b200.distributed.context import WorkerEnvironment
from shardtrain_b200.distributed.topology import Topology


def test_defaults_validate_in_reference_mode():
    Config().validate(1, mode="reference")


def test_reference_presets_load(tmp_path):
    preset = {
        "model": {"model_type": "qwen2", "vocab_size": 151936, "layers": 28, "hidden_size": 1536,
                  "num_heads": 12, "num_key_value_heads": 2, "mlp_hidden_size": 8960, "seq_len": 512},
        "parallel": {"fsdp_degree": 4, "tp_degree": 2, "sp_enabled": True, "device": "cuda", "backend": "nccl"},
        "runtime": {"param_grouping": "block", "reshard_after_forward": True, "forward_prefetch": True,
                    "backward_prefetch": True, "async_grad_rs": True, "communication_policy": "stream_ordered"},
        "training": {"dtype": "bf16", "optimizer": "adamw", "lr": 1e-5, "steps": 30,
                     "local_batch_size": 2, "accumulation_steps": 2},
    }
    path = tmp_path / "c.yaml"
    path.write_text(yaml.safe_dump(preset))
    cfg = load_config(path, ["--training.steps", "5", "--parallel.fsdp_degree", "8", "--parallel.tp_degree", "1",
                             "--parallel.sp_enabled", "false"])
    cfg.validate(8, mode="runtime")
    assert cfg.training.steps == 5 and cfg.parallel.strategy == "F8T1"


@pytest.mark.parametrize("patch,mode,fragment", [
    ({"parallel": {"fsdp_degree": 3}}, "runtime", "F=1/2/4/8"),
    ({"parallel": {"tp_degree": 2, "sp_enabled": True}, "model": {"seq_len": 15}}, "runtime", "seq_len"),
    ({"parallel": {"sp_enabled": True}}, "runtime", "SP requires"),
    ({"parallel": {"device": "cpu", "backend": "nccl"}}, "runtime", "Gloo"),
    ({"model": {"dropout": 0.1}}, "reference", "dropout"),
    ({"runtime": {"prefetch": "next"}}, "runtime", "forward_prefetch"),
    ({"runtime": {"forward_prefetch": True}}, "train", "Async"),
    ({"model": {"model_type": "qwen2"}}, "train", "runtime mode"),
    ({"training": {"accumulation_steps": 2}}, "runtime", "accumulation"),
    ({"runtime": {"communication_backend": "peer"}}, "runtime", "peer"),
])
def test_rejections(patch, mode, fragment):
    base = {"runtime": {"param_grouping": "block"}} if mode == "runtime" else {}
    for section, values in patch.items():
        base.setdefault(section, {}).update(values)
    cfg = config_from_dict(base)
    with pytest.raises(ConfigError, match=fragment):
        cfg.validate(cfg.parallel.world_size, mode=mode)


def test_strict_keys_types_and_overrides(tmp_path):
    with pytest.raises(ConfigError, match="Unknown config sections"):
        config_from_dict({"modle": {}})
    with pytest.raises(ConfigError, match="Unknown fields"):
        config_from_dict({"model": {"hiden": 1}})
    with pytest.raises(ConfigError, match="must be int"):
        config_from_dict({"model": {"layers": "2"}})
    assert config_from_dict({"training": {"lr": 1}}).training.lr == 1.0
    with pytest.raises(ConfigError, match="pairs"):
        load_config(None, ["--training.lr"])
    with pytest.raises(ConfigError, match="Invalid override"):
        load_config(None, ["training.lr=1", "x"])
    with pytest.raises(ConfigError, match="Unknown config field"):
        load_config(None, ["--training.nope", "1"])
    with pytest.raises(ConfigError, match="WORLD_SIZE=3"):
        Config().validate(3)
    # the sm_100a switches: defaults chosen by measurement, typed overrides, bad values refused
    runtime = Config().runtime
    assert (runtime.cuda_graphs, runtime.fused_allgather, runtime.fused_seq_gather, runtime.nvls,
            runtime.wire_dtype) == (True, "auto", False, "off", "bf16")
    assert load_config(None, ["--runtime.cuda_graphs", "false"]).runtime.cuda_graphs is False
    with pytest.raises(ConfigError, match="must be bool"):
        load_config(None, ["--runtime.cuda_graphs", "maybe"])
    for field, value in (("nvls", "on"), ("fused_allgather", "always"), ("wire_dtype", "fp16")):
        with pytest.raises(ConfigError, match=f"runtime.{field}"):
            load_config(None, [f"--runtime.{field}", value]).validate()


def test_strategy_names():
    assert parse_strategy("F4T2/SP") == (4, 2, True)
    assert parse_strategy("f8t1") == (8, 1, False)
    cfg = with_strategy(Config(), "F2T2/SP")
    assert cfg.parallel.world_size == 4 and cfg.parallel.strategy == "F2T2/SP"
    with pytest.raises(ConfigError):
        parse_strategy("DP8")


def test_topology_arithmetic():
    topo = Topology(4, 2)
    assert topo.world_size == 8
    assert [topo.coordinate(r) for r in (0, 1, 2, 7)] == [
        type(topo.coordinate(0))(0, 0), type(topo.coordinate(0))(0, 1),
        type(topo.coordinate(0))(1, 0), type(topo.coordinate(0))(3, 1)]
    assert topo.tp_groups == ((0, 1), (2, 3), (4, 5), (6, 7))
    assert topo.fsdp_groups == ((0, 2, 4, 6), (1, 3, 5, 7))
    assert all(topo.rank(*divmod(r, 2)) == r for r in range(8))
    roles = [role for role, _ in topo.creation_order]
    assert roles == ["tp"] * 4 + ["fsdp"] * 2 + ["tp_grad"] * 4 + ["fsdp_grad"] * 2
    assert topo.groups_for_rank(5) == {"tp": (4, 5), "fsdp": (1, 3, 5, 7), "tp_grad": (4, 5),
                                       "fsdp_grad": (1, 3, 5, 7)}
    for bad in (lambda: Topology(0, 1), lambda: topo.coordinate(8), lambda: topo.rank(4, 0)):
        with pytest.raises(ValueError):
            bad()


def test_worker_environment():
    assert WorkerEnvironment.read({}) == WorkerEnvironment()
    env = WorkerEnvironment.read({"RANK": "3", "LOCAL_RANK": "1", "WORLD_SIZE": "4"})
    assert (env.rank, env.local_rank, env.world_size, env.launched) == (3, 1, 4, True)
    for bad in ({"RANK": "0"}, {"RANK": "x", "LOCAL_RANK": "0", "WORLD_SIZE": "1"},
                {"RANK": "2", "LOCAL_RANK": "0", "WORLD_SIZE": "2"}):
        with pytest.raises(ConfigError):
            WorkerEnvironment.read(bad)
