import copy
import json

import pytest
import torch

from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
from shardtrain_b200.models.qwen2_checkpoint import (CheckpointError, QwenCheckpoint, SafetensorsFile,
                                                     load_qwen_checkpoint, save_safetensors)
from shardtrain_b200.runtime.checkpoint import (full_state_dict, load_full_optimizer, load_sharded,
                                                save_full, save_sharded)
from shardtrain_b200.runtime.engine import ShardedRuntime
from shardtrain_b200.training.qwen2_trainer import QwenTrainer

CFG = Qwen2ModelConfig(vocab_size=256, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2)


def trained(steps=2, seed=0):
    torch.manual_seed(seed)
    model = Qwen2CausalLM(CFG)
    rt = ShardedRuntime(device="cpu")
    rt.register(model)
    tr = QwenTrainer(model, rt, lr=1e-3, optimizer="adamw")
    for s in range(steps):
        tr.train_step(torch.randint(0, 256, (2, 8), generator=torch.Generator().manual_seed(s)))
    return model, rt, tr


def test_safetensors_roundtrip_and_slices(tmp_path):
    tensors = {"a": torch.arange(12.).view(3, 4), "b": torch.ones(5, dtype=torch.bfloat16),
               "c": torch.tensor(3, dtype=torch.int64)}
    save_safetensors(tmp_path / "x.safetensors", tensors, {"k": "v"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert f.metadata == {"k": "v"}
    for k, v in tensors.items():
        assert torch.equal(f.tensor(k), v)
    assert torch.equal(f.rows("a", 1, 2), tensors["a"][1:3])
    # the file is readable by the reference ecosystem's parser too
    from safetensors import safe_open
    with safe_open(str(tmp_path / "x.safetensors"), framework="pt") as h:
        assert torch.equal(h.get_tensor("a"), tensors["a"])


def test_strict_reader_rejections(tmp_path):
    save_safetensors(tmp_path / "model.safetensors", {"w": torch.zeros(2, 2), "extra": torch.zeros(1)})
    with pytest.raises(CheckpointError, match="Unexpected keys: extra"):
        QwenCheckpoint(tmp_path, {"w": (2, 2)})
    with pytest.raises(CheckpointError, match="Missing keys"):
        QwenCheckpoint(tmp_path, {"w": (2, 2), "extra": (1,), "gone": (1,)})
    with pytest.raises(CheckpointError, match="Shape mismatches"):
        QwenCheckpoint(tmp_path, {"w": (4,), "extra": (1,)})
    with pytest.raises(CheckpointError, match="does not exist"):
        QwenCheckpoint(tmp_path / "nope")
    idx = tmp_path / "idx"
    idx.mkdir()
    save_safetensors(idx / "s1.safetensors", {"w": torch.zeros(1), "hidden": torch.zeros(1)})
    (idx / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "s1.safetensors"}}))
    with pytest.raises(CheckpointError, match="absent from the index"):
        QwenCheckpoint(idx)
    (idx / "model.safetensors.index.json").write_text('{"weight_map": {"w": "../x.safetensors"}}')
    with pytest.raises(CheckpointError, match="escapes|Missing or unsupported"):
        QwenCheckpoint(idx)
    (idx / "model.safetensors.index.json").write_text('{"weight_map": {"w": "a"}, "weight_map": {}}')
    with pytest.raises(CheckpointError, match="Duplicate JSON key"):
        QwenCheckpoint(idx)
    with pytest.raises(CheckpointError, match="tied_aliases require"):
        QwenCheckpoint(tmp_path, None, {"a": "b"})


def test_dense_loader_and_tied_alias(tmp_path):
    torch.manual_seed(1)
    src = Qwen2CausalLM(CFG)
    state = {k: v.detach().clone() for k, v in src.state_dict().items() if k != "lm_head.weight"}
    save_safetensors(tmp_path / "model.safetensors", state)
    dst = Qwen2CausalLM(CFG)
    report = load_qwen_checkpoint(dst, tmp_path)
    assert report.omitted_tied_aliases == ("lm_head.weight",)
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n


def test_sharded_resume_is_bit_exact(tmp_path):
    model, rt, tr = trained()
    save_sharded(rt, tmp_path, tr.optimizer, trainer_step=tr.step_id)
    ids = torch.randint(0, 256, (2, 8), generator=torch.Generator().manual_seed(9))
    expected = tr.train_step(ids).loss
    after = {n: h.local_shard.detach().clone() for n, h in rt.registry.items()}
    model2, rt2, tr2 = trained(steps=0, seed=5)
    meta = load_sharded(rt2, tmp_path, tr2.optimizer)
    assert meta["optimizer_step"] == 2 and tr2.optimizer.arena_step == 2
    assert tr2.train_step(ids).loss == expected
    for n, h in rt2.registry.items():
        assert torch.equal(h.local_shard, after[n]), n


def test_full_export_reloads_through_the_strict_reader(tmp_path):
    model, rt, tr = trained()
    save_full(rt, tmp_path, tr.optimizer)
    full = full_state_dict(rt)
    assert full["model.layers.0.self_attn.q_proj.weight"].shape == (32, 32)
    fresh = Qwen2CausalLM(CFG, device="meta", dtype=torch.float32)
    fresh._qwen_weight_source = QwenCheckpoint(tmp_path)
    rt2 = ShardedRuntime(device="cpu")
    rt2.register(fresh)
    tr2 = QwenTrainer(fresh, rt2, lr=1e-3, optimizer="adamw")
    load_full_optimizer(rt2, tmp_path, tr2.optimizer)
    for n, h in rt.registry.items():
        assert torch.equal(rt2.registry[n].local_shard, h.local_shard), n
    assert torch.equal(tr2.optimizer.exp_avg_sq, tr.optimizer.exp_avg_sq)
    ids = torch.randint(0, 256, (2, 8), generator=torch.Generator().manual_seed(9))
    assert tr2.train_step(ids).loss == tr.train_step(ids).loss


def test_failed_runtime_refuses_to_save(tmp_path):
    model, rt, tr = trained(steps=1)
    rt.fail("injected")
    with pytest.raises(RuntimeError, match="FAILED runtime"):
        save_sharded(rt, tmp_path, tr.optimizer)
    with pytest.raises(RuntimeError, match="FAILED runtime"):
        save_full(rt, tmp_path, tr.optimizer)


def test_sharded_load_restores_the_step_counters(tmp_path):
    model, rt, tr = trained()
    save_sharded(rt, tmp_path, tr.optimizer, trainer=tr)
    model2, rt2, tr2 = trained(steps=0, seed=5)
    meta = load_sharded(rt2, tmp_path, tr2.optimizer, trainer=tr2)
    assert tr2.step_id == tr.step_id == 2 and rt2.step_id == rt.step_id == meta["runtime_step"]
    assert all(float(s["step"]) == 2.0 for s in tr2.optimizer.state.values())
    assert tr2.train_step(torch.randint(0, 256, (2, 8))).step == 2


@pytest.mark.distributed
def test_two_rank_save_reloads_on_one_and_four_ranks(tmp_path):
    """Save on F2 (gloo), reload the canonical export on F1 and F4: parameters and AdamW moments
    are pure data movement (bit-equal), and the next step's loss on the same global batch agrees
    to float tolerance; the sharded format resumes on the same mesh bit-exactly."""
    import json

    from tests.launch import run_workers

    from shardtrain_b200.models.qwen2_checkpoint import SafetensorsFile

    def run(mode, fsdp):
        code, log = run_workers("tests.workers.checkpoint_worker", fsdp,
                                ["--dir", tmp_path, "--mode", mode, "--fsdp", fsdp])
        assert code == 0, log[-3000:]
        state = SafetensorsFile(tmp_path / f"state.{mode}.f{fsdp}.safetensors")
        loss = json.loads((tmp_path / f"loss.{mode}.f{fsdp}.json").read_text())["loss"]
        return state, loss

    saved, saved_loss = run("save", 2)
    names = list(saved.entries)
    assert any(n.startswith("exp_avg_sq.") for n in names)
    for mode, fsdp in (("load", 1), ("load", 4), ("load_sharded", 2)):
        state, loss = run(mode, fsdp)
        for name in names:
            assert torch.equal(state.tensor(name), saved.tensor(name)), (mode, fsdp, name)
        assert loss == pytest.approx(saved_loss, rel=(0 if mode == "load_sharded" else 2e-6))


def test_checkpoint_oracle_tool_compares_dense_and_runtime_and_changes_nothing(tmp_path, capsys):
    """`utils.verify_checkpoint`: a tiny random HF-named checkpoint passes (loss and every
    parameter gradient of the runtime equal the dense model's, shards untouched); a checkpoint
    with one tensor missing is refused before anything runs."""
    import json

    import yaml

    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.utils import verify_checkpoint

    torch.manual_seed(3)
    cfg = Qwen2ModelConfig(vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=True)
    dense = Qwen2CausalLM(cfg)
    tensors = {n: p.detach().clone() for n, p in dense.named_parameters()}
    good = tmp_path / "good"
    good.mkdir()
    save_safetensors(good / "model.safetensors", tensors)
    config_file = tmp_path / "config.yaml"
    config_file.write_text(yaml.safe_dump(cfg.to_dict()))
    code = verify_checkpoint.main(["--checkpoint", str(good), "--hf-config", str(config_file),
                                   "--batch", "2", "--seq-len", "12"])
    printed = capsys.readouterr().out
    report = json.loads(printed[printed.index("{"):])
    assert code == 0 and report["passed"] and not report["problems"]
    assert report["parameters"] == sum(t.numel() for t in tensors.values())
    assert report["loss_runtime"] == pytest.approx(report["loss_dense"], rel=1e-5)
    assert report["worst_gradient"]["relative_to_max"] < 1e-4 and len(report["shard_sha256"]) == 64
    bad = tmp_path / "bad"
    bad.mkdir()
    fewer = dict(tensors)
    fewer.pop("model.norm.weight")
    save_safetensors(bad / "model.safetensors", fewer)
    with pytest.raises(CheckpointError, match="Missing keys"):
        verify_checkpoint.main(["--checkpoint", str(bad), "--hf-config", str(config_file)])
