"""Fused sm_100a executor end to end on one GPU against the dense model (run with -m gpu)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def build(tied, accumulate=2, optimizer="sgd", lr=0.05, retain=False, graphs=True):
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
                        retain_parameters=retain, cuda_graphs=graphs)
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
        # no single element may be far off either (a misplaced row or column would show here
        # long before it moves the norm): bf16 rounding noise stays a small fraction of the scale
        worst = (grad - p.grad).abs().max() / (p.grad.abs().max() + 1e-12)
        assert worst < 8e-2, (name, worst.item())
    assert all(p.ndim == 1 and p.dtype == torch.float32 for p in model.parameters())
    assert not rt.comm.live_buffers


def test_replayed_layer_graphs_give_the_same_bits_as_kernel_by_kernel_launches():
    """A layer's launch sequence is captured the second time its arguments repeat and replayed
    afterwards: five AdamW steps must end in exactly the same shards and losses as with every
    kernel launched by itself, graphs must actually have been built, and a changed input shape
    (other keys) must keep working."""
    from shardtrain_b200 import ops

    stb = ops.load()
    stb.replay_clear()
    batches = [torch.randint(0, 2048, (4, 256), device="cuda") for _ in range(5)]   # new data each step
    runs = {}
    for graphs in (False, True):
        # SGD: a parameter moves in proportion to its gradient, so the run-to-run rounding noise of
        # the embedding's atomic scatter-add stays rounding noise (AdamW's g / sqrt(v) would turn
        # it into whole steps for elements whose gradient is nearly zero)
        dense, model, rt, tr = build(True, optimizer="sgd", lr=0.05, graphs=graphs)
        before = int(stb.launch_count())
        losses = [tr.train_step(ids).loss for ids in batches]
        torch.cuda.synchronize()
        ops.check_status("replay")
        runs[graphs] = (losses, [p.detach().clone() for p in model.parameters()],
                        int(stb.launch_count()) - before)
        if graphs:
            # 2 layers x (forward + backward with 2 gradient-slot rotations) at least
            assert int(stb.replay_graphs()) >= 4
            shorter = torch.randint(0, 2048, (4, 128), device="cuda")
            assert tr.train_step(shorter).loss > 0          # new shapes: new keys, no stale replay
            torch.cuda.synchronize()
            ops.check_status("replay, second shape")
        else:
            assert int(stb.replay_graphs()) == 0
    # (the embedding's scatter-add uses atomics, so two runs agree to rounding, not to the bit)
    assert runs[True][0] == pytest.approx(runs[False][0], rel=1e-4)
    for a, b in zip(runs[True][1], runs[False][1]):
        torch.testing.assert_close(a, b, atol=2e-5, rtol=1e-4)
    assert runs[True][2] == runs[False][2]                 # replayed kernels are counted too
    stb.replay_clear()


def test_fresh_mask_and_position_tensors_every_step_still_hit_the_replay_cache():
    """A training loop builds new mask / position tensors every step.  Their packed bits and RoPE
    tables live at fixed addresses, so the layers' replay keys repeat exactly as they do when one
    mask tensor is reused: the same number of graphs (bounded by layers x gradient slots), and
    the same masked result."""
    from shardtrain_b200 import ops

    stb = ops.load()
    ids = torch.randint(0, 2048, (4, 256), device="cuda")

    def inputs():
        mask = torch.ones_like(ids)
        mask[1, 200:] = 0                                     # one padded sample
        return mask, torch.arange(256, device="cuda").unsqueeze(0).clone()

    losses, graphs = {}, {}
    for fresh in (True, False):
        stb.replay_clear()
        dense, model, rt, tr = build(True, optimizer="sgd", lr=0.05)
        kept = inputs()
        run = []
        for step in range(6):
            mask, positions = inputs() if fresh else kept
            run.append(tr.train_step(ids, ids, attention_mask=mask, position_ids=positions).loss)
        torch.cuda.synchronize()
        ops.check_status("fresh inputs")
        losses[fresh], graphs[fresh] = run, int(stb.replay_graphs())
    # 2 layers: one forward sequence each, one backward sequence per gradient slot (4) at most
    assert 4 <= graphs[True] == graphs[False] <= 2 + 2 * 4
    # (a wrong or stale mask moves the loss by percents; atomics in the embedding's scatter-add
    # move it by rounding noise)
    assert losses[True] == pytest.approx(losses[False], rel=1e-3)
    stb.replay_clear()


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


def _small_model(seed=0, tied=True):
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig

    torch.manual_seed(seed)
    cfg = Qwen2ModelConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                           num_attention_heads=2, num_key_value_heads=1, tie_word_embeddings=tied)
    return Qwen2CausalLM(cfg).cuda()


@pytest.mark.parametrize("backend,dtype", [("nccl", "fp32"), ("auto", "fp32"), ("nccl", "bf16")])
def test_portable_executor_on_cuda_follows_the_configured_dtype(backend, dtype):
    """`communication_backend: nccl`, or a compute dtype the sm_100a kernels do not have, selects
    the portable executor on CUDA (five streams, torch ops); fp32 then matches the dense model to
    fp32 tolerance instead of silently training in bf16."""
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    dense = _small_model()
    model = copy.deepcopy(dense)
    rt = ShardedRuntime(device="cuda:0", reshard_after_forward=True, forward_prefetch=True,
                        backward_prefetch=True, async_grad_rs=True,
                        communication_policy="conservative", communication_backend=backend,
                        compute_dtype=dtype).register(model)
    assert rt.executor.name == "portable" and rt.fused is None
    assert len(rt.comm.streams) == 5
    tr = QwenTrainer(model, rt, lr=0.05, dtype=dtype, optimizer="sgd", accumulation_steps=2)
    opt = torch.optim.SGD(dense.parameters(), lr=0.05)
    ids = torch.randint(0, 2048, (4, 128), device="cuda")
    for _ in range(2):
        got = tr.train_step(ids)
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == "bf16"):
            want = dense(ids, labels=ids).loss
        want.backward()
        opt.step()
        assert got.loss == pytest.approx(want.item(), rel=2e-5 if dtype == "fp32" else 2e-3)
    full = rt.reconstruct_tp_local()
    tol = 2e-5 if dtype == "fp32" else 2e-3
    for name, p in dense.named_parameters():
        torch.testing.assert_close(full[name], p.detach(), atol=tol, rtol=tol)
    assert not rt.comm.live_buffers


def test_trainer_refuses_a_dtype_the_fused_executor_does_not_compute_in():
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    model = _small_model()
    rt = ShardedRuntime(device="cuda:0").register(model)        # dtype not stated: sm_100a executor
    assert rt.executor.name == "fused"
    with pytest.raises(ValueError, match="bf16 only"):
        QwenTrainer(model, rt, lr=0.05, dtype="fp32", optimizer="sgd")


def test_fp16_overflow_skips_the_update_and_recovers():
    """fp16 AMP on CUDA (portable executor): an inf written into one shard gradient on the host
    makes the step an overflow -- no parameter moves, the loss scale backs off, the growth
    tracker restarts -- and the next step trains normally with the smaller scale
    (behaviour of tests/cuda/test_qwen2_amp.py:210-308 of the reference)."""
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    model = _small_model(seed=4)
    rt = ShardedRuntime(device="cuda:0", reshard_after_forward=True, compute_dtype="fp16").register(model)
    assert rt.executor.name == "portable"
    tr = QwenTrainer(model, rt, lr=1e-3, dtype="fp16", optimizer="adamw")
    ids = torch.randint(0, 2048, (2, 128), device="cuda")
    first = tr.train_step(ids)
    assert not first.overflow and first.loss_scale == 128.0
    before = rt.param_arena.clone()
    moments = tr.optimizer.exp_avg.clone()
    finalize, armed = rt.finalize_backward, {"on": True}

    def poisoned(*args, **kwargs):
        if armed.pop("on", False):
            rt.grad_arena[5] = float("inf")          # host-side injection, no kernel faults
        return finalize(*args, **kwargs)

    rt.finalize_backward = poisoned
    skipped = tr.train_step(ids)
    assert skipped.overflow and skipped.loss_scale == 64.0
    assert torch.equal(rt.param_arena, before) and torch.equal(tr.optimizer.exp_avg, moments)
    assert tr.optimizer.arena_step == 1 and not rt.failed
    after = tr.train_step(ids)
    assert not after.overflow and after.loss_scale == 64.0
    assert not torch.equal(rt.param_arena, before) and tr.optimizer.arena_step == 2
    assert after.loss == after.loss           # finite


def test_sharded_checkpoint_reload_rebuilds_the_bf16_shadow(tmp_path):
    """The fused executor gathers matrices from a bf16 shadow of the shards.  Loading a
    checkpoint rewrites the FP32 masters behind its back: the shadow must be marked stale and
    rebuilt before the next gather, so the step after a reload repeats the original one."""
    from shardtrain_b200.runtime.checkpoint import load_sharded, save_sharded

    dense, model, rt, tr = build(True, optimizer="adamw", lr=1e-3)
    ids = torch.randint(0, 2048, (4, 256), device="cuda")
    tr.train_step(ids)
    save_sharded(rt, tmp_path, tr.optimizer, trainer=tr)
    saved = rt.param_arena.clone()
    want = tr.train_step(ids).loss
    tr.train_step(ids)                                   # move further away from the checkpoint
    load_sharded(rt, tmp_path, tr.optimizer, trainer=tr)
    assert rt.fused._shadow_stale and torch.equal(rt.param_arena, saved)
    got = tr.train_step(ids)
    assert got.step == 1 and got.loss == pytest.approx(want, rel=1e-5)
    assert torch.equal(rt.fused.shadow.float(), rt.param_arena.bfloat16().float())
