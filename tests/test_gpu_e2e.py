"""Fused sm_100a executor end to end on one GPU against the dense model (run with -m gpu)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def build(tied, accumulate=2, optimizer="sgd", lr=0.05, retain=False):
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    torch.manual_seed(0)
    cfg = Qwen2ModelConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                           num_attention_heads=2, num_key_value_heads=1, tie_word_embeddings=tied)
    dense = Qwen2CausalLM(cfg).cuda()
    model = copy.deepcopy(dense)
    rt = ShardedRuntime(device="cuda:0", reshard_after_forward=True, forward_prefetch=True,
                        backward_prefetch=True, async_grad_rs=True, communication_policy="stream_ordered",
                        retain_parameters=retain)
    rt.register(model)
    assert rt.executor.name == "fused"
    tr = QwenTrainer(model, rt, lr=lr, dtype="bf16", optimizer=optimizer, accumulation_steps=accumulate)
    return dense, model, rt, tr


@pytest.mark.parametrize("tied", [True, False])
def test_gradients_match_dense_bf16_autocast(tied):
    from shardtrain_b200 import ops

    dense, model, rt, tr = build(tied)
    ids = torch.randint(0, 2048, (4, 256), device="cuda")
    before = {n: p.detach().clone() for n, p in dense.named_parameters()}
    got = tr.train_step(ids)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = dense(ids, labels=ids)
    out.loss.backward()
    assert got.loss == pytest.approx(out.loss.item(), rel=2e-3)
    assert got.valid_tokens == 4 * 255
    torch.cuda.synchronize()
    ops.check_status("e2e")
    full = rt.reconstruct_tp_local()
    # one SGD step: (before - after) / lr is the gradient; compare with the dense bf16 gradient
    for name, p in dense.named_parameters():
        grad = (before[name] - full[name]) / 0.05
        err = (grad - p.grad).norm() / (p.grad.norm() + 1e-12)
        assert err < 3e-2, (name, err.item())
    assert all(p.ndim == 1 and p.dtype == torch.float32 for p in model.parameters())
    assert not rt.comm.live_buffers


@pytest.mark.parametrize("retain", [False, True])
def test_adamw_training_reduces_loss_and_fuses_the_update(retain):
    from shardtrain_b200 import ops

    dense, model, rt, tr = build(True, optimizer="adamw", lr=1e-3, retain=retain)
    assert tr.optimizer.fuse_into_reduction
    ids = torch.randint(0, 2048, (4, 256), device="cuda")
    losses = [tr.train_step(ids).loss for _ in range(6)]
    torch.cuda.synchronize()
    ops.check_status("e2e adamw")
    assert losses[-1] < losses[0] - 0.05
    kinds = [t.kind for t in rt.comm.tickets]
    assert "fsdp_rs_accumulate_adamw" in kinds and "fsdp_ag_cast" in kinds
    per_micro = 2 * 2 + 2
    gathers = kinds.count("fsdp_ag_cast")
    assert gathers == (6 * 2 * per_micro if not retain else 6 * (2 + 2))


def test_caller_supplied_position_ids_match_default_positions():
    """Explicit positions 0..S-1, as one shared row and per sample, give the loss of the default;
    stretched positions change it."""
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    torch.manual_seed(3)
    cfg = Qwen2ModelConfig(vocab_size=512, hidden_size=256, intermediate_size=512,
                           num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1)
    model = Qwen2CausalLM(cfg)
    rt = ShardedRuntime(device="cuda").register(model)
    trainer = QwenTrainer(model, rt, lr=0.0, dtype="bf16", optimizer="sgd")
    ids = torch.randint(0, 512, (2, 128), device="cuda")
    base = trainer.train_step(ids).loss
    row = torch.arange(128, device="cuda").unsqueeze(0)
    assert trainer.train_step(ids, position_ids=row).loss == pytest.approx(base, rel=1e-6)
    assert trainer.train_step(ids, position_ids=row.expand(2, -1).contiguous()).loss == \
        pytest.approx(base, rel=1e-6)
    # a constant shift would not do: rotary attention depends on position differences only
    assert abs(trainer.train_step(ids, position_ids=row * 3).loss - base) > 1e-4


def test_expired_device_wait_fails_the_step_on_the_host():
    """A bounded device-side wait that gave up (here: a barrier whose peer flag nobody sets, with a
    tiny spin limit) is seen by the trainer in the same read as the step metrics: the step
    raises, the runtime goes FAILED, the CUDA context stays usable."""
    from shardtrain_b200 import ops as module

    dense, model, rt, tr = build(True)
    ids = torch.randint(0, 2048, (4, 128), device="cuda")
    tr.train_step(ids)
    pads = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(2)]
    module.load().peer_barrier([p.data_ptr() for p in pads], 0, 3, 1, 1000)   # "peer 1" is silent
    with pytest.raises(RuntimeError, match="peer flag wait expired"):
        tr.train_step(ids)
    assert rt.failed
    with pytest.raises(RuntimeError):
        tr.train_step(ids)
    assert module.load().status_read() == 0
    assert torch.ones(8, device="cuda").sum().item() == 8


def test_nonfinite_gradient_is_caught_by_the_reduction_kernels_check():
    """An inf slipped into the gradient arena between the two micro-steps (host-side injection)
    reaches the second reduce-scatter's accumulate, whose built-in check flags it; the step
    raises and the runtime is FAILED."""
    dense, model, rt, tr = build(True, accumulate=2, optimizer="adamw", lr=1e-3)
    ids = torch.randint(0, 2048, (4, 128), device="cuda")
    tr.train_step(ids)
    end_step, state = rt.end_step, {"armed": True}

    def poisoned_end_step():
        end_step()
        if state.pop("armed", False):
            rt.grad_arena[3] = float("inf")

    rt.end_step = poisoned_end_step
    with pytest.raises(RuntimeError, match="Nonfinite"):
        tr.train_step(ids)
    assert rt.failed
