"""Single-process (degree-1) runtime: every lifecycle rule is enforced without a process group."""
import copy
import itertools
import weakref

import pytest
import torch

from shardtrain_b200.config import ModelConfig
from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
from shardtrain_b200.models.reference import build_reference_model, synthetic_batch
from shardtrain_b200.runtime.engine import ShardedRuntime
from shardtrain_b200.training.qwen2_trainer import QwenTrainer
from shardtrain_b200.training.reference import dense_oracle
from shardtrain_b200.training.sharded_trainer import ShardedTrainer

TOY = ModelConfig(layers=3, hidden_size=32, num_heads=4, mlp_hidden_size=64, seq_len=8)


def tiny_qwen(tied=True):
    return Qwen2ModelConfig(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=tied)


@pytest.mark.parametrize("policy", ["conservative", "stream_ordered"])
@pytest.mark.parametrize("flags", list(itertools.product([False, True], repeat=3)))
def test_toy_matches_dense_for_every_switch_combination(flags, policy):
    dense = build_reference_model(TOY, 3)
    model = copy.deepcopy(dense)
    fp, bp, ar = flags
    rt = ShardedRuntime(device="cpu", reshard_after_forward=True, forward_prefetch=fp,
                        backward_prefetch=bp, async_grad_rs=ar, communication_policy=policy)
    rt.register(model)
    trainer = ShardedTrainer(model, rt, 0.1)
    ref = torch.optim.SGD(dense.parameters(), lr=0.1)
    for step in range(3):
        x = synthetic_batch(TOY, 4, step)
        got = trainer.train_step(x, torch.zeros_like(x))
        ref.zero_grad()
        loss = dense(x).square().mean()
        loss.backward()
        ref.step()
        assert got.loss == pytest.approx(loss.item(), rel=1e-6)
    full = rt.reconstruct_tp_local()
    for name, p in dense.named_parameters():
        torch.testing.assert_close(full[name], p, atol=3e-6, rtol=3e-5)
    per_step = rt.comm.events.count  # noqa: B018 - events exist
    materialized = [e for e in rt.comm.events if e["event_type"] == "materialize_issue"]
    assert len(materialized) == 3 * (TOY.layers + TOY.layers - 1)   # no BWD gather for the last unit
    assert not rt.comm.live_buffers


def test_toy_output_matches_functional_oracle():
    dense = build_reference_model(TOY, 5)
    params = {n: p.detach().clone() for n, p in dense.named_parameters()}
    x = synthetic_batch(TOY, 2, 0)
    torch.testing.assert_close(dense(x), dense_oracle(x, params, TOY)[-1], atol=2e-6, rtol=2e-5)


def test_no_full_parameter_is_saved_for_backward():
    dense = Qwen2CausalLM(tiny_qwen())
    model = copy.deepcopy(dense)
    rt = ShardedRuntime(device="cpu", reshard_after_forward=True)
    rt.register(model)
    rt.compute_dtype = torch.float32
    weight_shapes = {h.spec.tp_local_shape for h in rt.registry.values() if len(h.spec.tp_local_shape) == 2}
    full_storages, saved = set(), []
    original = rt.comm.buffer

    def tracking_buffer(tensor, owner):
        if owner == "full_parameter":
            full_storages.add(tensor.untyped_storage().data_ptr())
        return original(tensor, owner)

    rt.comm.buffer = tracking_buffer

    def pack(t):
        saved.append((tuple(t.shape), t.untyped_storage().data_ptr()))
        return t

    ids = torch.randint(0, 1024, (2, 16))
    rt.begin_step(0)
    rt.zero_grad()
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        out = model(ids, labels=ids)
    assert full_storages and saved
    # freed storages can be reused by later activations, so pointer identity is only meaningful
    # for the full parameters that are still alive (retained units)
    alive = {l.tensor.untyped_storage().data_ptr() for l in rt.comm.live_buffers.values()
             if l.owner == "full_parameter"}
    assert alive
    assert not any(ptr in alive for _, ptr in saved)
    assert not any(shape in weight_shapes for shape, _ in saved)
    out.loss.backward()
    rt.finalize_backward()
    assert not rt.comm.live_buffers


@pytest.mark.parametrize("tied", [True, False])
@pytest.mark.parametrize("reshard", [True, False])
def test_qwen_sgd_parity_and_state_layout(tied, reshard):
    torch.manual_seed(0)
    dense = Qwen2CausalLM(tiny_qwen(tied))
    model = copy.deepcopy(dense)
    rt = ShardedRuntime(device="cpu", reshard_after_forward=reshard, forward_prefetch=True,
                        backward_prefetch=True)
    rt.register(model)
    trainer = QwenTrainer(model, rt, lr=0.05, optimizer="sgd", accumulation_steps=2)
    ref = torch.optim.SGD(dense.parameters(), lr=0.05)
    for step in range(3):
        ids = torch.randint(0, 1024, (4, 16), generator=torch.Generator().manual_seed(step))
        got = trainer.train_step(ids)
        ref.zero_grad()
        out = dense(ids, labels=ids)
        out.loss.backward()
        ref.step()
        assert got.loss == pytest.approx(out.loss.item(), rel=2e-6)
        assert got.valid_tokens == 4 * 15
    full = rt.reconstruct_tp_local()
    for name, p in dense.named_parameters():
        torch.testing.assert_close(full[name], p, atol=3e-6, rtol=3e-5)
    # HF names survive, every value is this rank's flat FP32 shard, tied head aliases the embedding
    names = dict(model.named_parameters())
    assert set(names) == set(dict(dense.named_parameters()))
    assert all(p.ndim == 1 and p.dtype == torch.float32 for p in names.values())
    assert (model.lm_head.weight is model.model.embed_tokens.weight) == tied
    assert len(rt.units) == (4 if tied else 5)
    # tied: L+2 forward, L backward (unit 0 and the last unit stay materialised)
    # untied: L+3 forward, L+2 backward (only the head, the last unit, is retained)
    per_step = 2 * 2 + 2 if tied else 2 * 2 + 5
    issued = [e for e in rt.comm.events if e["event_type"] == "materialize_issue"]
    if reshard:
        assert len(issued) == 3 * 2 * per_step


def test_step_protocol_guards():
    dense = Qwen2CausalLM(tiny_qwen())
    rt = ShardedRuntime(device="cpu")
    rt.register(dense)
    trainer = QwenTrainer(dense, rt, optimizer="sgd")
    with pytest.raises(ValueError, match="exactly the persistent local shards"):
        rt.bind_optimizer(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1))
    with pytest.raises(RuntimeError, match="Premature optimizer"):
        trainer.optimizer.step()
    with pytest.raises(RuntimeError, match="Invalid step boundary"):
        rt.begin_step(5)
    rt.begin_step(0)
    with pytest.raises(RuntimeError, match="Invalid step boundary"):
        rt.begin_step(1)
    with pytest.raises(RuntimeError, match="Missing gradient readiness"):
        rt.finalize_backward()
    rt.fail("test")
    assert all(u.state == "FAILED" for u in rt.units)
    rt.active = False
    with pytest.raises(RuntimeError, match="FAILED runtime"):
        rt.begin_step(1)
    with pytest.raises(RuntimeError, match="already registered"):
        rt.register(dense)


def test_nonzero_padding_and_nonfinite_gradients_are_rejected():
    torch.manual_seed(0)
    model = Qwen2CausalLM(tiny_qwen())
    rt = ShardedRuntime(device="cpu")
    rt.register(model)
    trainer = QwenTrainer(model, rt, optimizer="sgd")
    ids = torch.randint(0, 1024, (2, 16))
    trainer.train_step(ids)
    handle = next(iter(rt.registry.values()))
    rt.begin_step(rt.step_id + 1)
    rt.zero_grad()
    model(ids, labels=ids).loss.backward()
    handle.grad_shard[0] = float("nan")
    with pytest.raises(RuntimeError, match="Nonfinite gradient"):
        rt.finalize_backward()


def test_executor_selection_rules(monkeypatch, caplog):
    """`auto` hands a run to the sm_100a executor only when that executor can serve it (bf16,
    head_dim 128, at most 8 ranks on one host); otherwise it falls back to the portable one and
    says why.  An explicit `peer` that cannot be met is an error, never a silent fallback."""
    from types import SimpleNamespace

    import torch.distributed as dist

    from shardtrain_b200 import ops
    from shardtrain_b200.runtime import qwen2_adapter as qa

    monkeypatch.setattr(ops, "available", lambda: True)

    def pick(backend="auto", dtype=None, head_dim=128, device="cuda", mesh=None):
        rt = SimpleNamespace(device=torch.device(device), communication_backend=backend,
                             requested_dtype=dtype)
        return qa._choose_executor(rt, SimpleNamespace(head_dim=head_dim), mesh)

    assert pick() == "fused" and pick(dtype="bf16") == "fused" and pick("peer") == "fused"
    assert pick("nccl") == "portable" and pick(device="cpu") == "portable"
    for kwargs, word in ((dict(dtype="fp32"), "fp32"), (dict(dtype="fp16"), "fp16"),
                         (dict(head_dim=64), "head_dim 64")):
        caplog.clear()
        with caplog.at_level("WARNING", logger="shardtrain_b200"):
            assert pick(**kwargs) == "portable"
        assert word in caplog.text
        with pytest.raises(ValueError, match="peer cannot serve"):
            pick("peer", **kwargs)
    with pytest.raises(ValueError, match="needs a CUDA device"):
        pick("peer", device="cpu")
    # meshes beyond the peer tables or spanning hosts
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 16)
    monkeypatch.setattr(qa, "_single_host", lambda: True)
    assert pick(mesh=object()) == "portable"
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 8)
    assert pick(mesh=object()) == "fused"
    monkeypatch.setattr(qa, "_single_host", lambda: False)
    assert pick(mesh=object()) == "portable"
    with pytest.raises(ValueError, match="several hosts"):
        pick("peer", mesh=object())


def test_runtime_rejects_an_unknown_compute_dtype():
    with pytest.raises(ValueError, match="compute_dtype"):
        ShardedRuntime(device="cpu", compute_dtype="int8")


def _dispatch_fixture():
    """Four bare units in the state the gradient-dispatch schedule expects when unit 3 (the last)
    is reducing: unit 3 entered backward and seeded the gather of unit 2; units 0..2 wait."""
    from shardtrain_b200.runtime.engine import UnitState
    from shardtrain_b200.runtime.materializer import MaterializationLease

    rt = ShardedRuntime(device="cpu", backward_prefetch=True, async_grad_rs=True,
                        communication_policy="stream_ordered")
    rt.sp = True
    assert rt.gradient_dispatch_prefetch
    issued = []

    def fake_prefetch(unit_id, phase):
        unit = rt.units[unit_id]
        issued.append((unit_id, phase))
        if unit.lease is None:
            unit.generation += 1
            unit.lease = MaterializationLease(unit_id, rt.step_id, phase, unit.generation)
            unit.state = f"{phase}_MATERIALIZING"

    rt.prefetch = fake_prefetch
    for uid in range(4):
        unit = UnitState(rt, uid, None)
        unit.forward_calls, unit.generation, unit.state = 1, 1, "RESHARDED"
        rt.units.append(unit)
    rt.step_id, rt.active = 0, True
    rt.backward_entry_expected = rt.backward_dispatch_expected = 3
    last = rt.units[3]
    last.state, last.lease = "FWD_RETAINED", MaterializationLease(3, 0, "FWD", 1)
    rt.validate_backward_prefetch_entry(last)
    last.backward_calls, last.state = 1, "BWD_ACTIVE"
    rt.backward_prefetch_entered(last)             # seeds the gather of unit 2
    assert issued == [(2, "BWD")] and rt.backward_entry_expected == 2
    last.reductions, last.state = 1, "GRAD_REDUCING"
    return rt, issued


def test_gradient_dispatch_issues_exactly_the_unit_two_below_the_owner():
    rt, issued = _dispatch_fixture()
    rt.dispatch_backward_prefetch(rt.units[3])
    assert issued == [(2, "BWD"), (1, "BWD")] and rt.backward_dispatch_expected == 2
    token = rt.backward_prefetch_tokens[(0, 2)]
    assert (token["target_unit"], token["gradient_owner"], token["status"]) == (1, 3, "issued")
    assert token["scheduling_boundary"] == "previous_gradient_dispatch"
    # unit 2 may now enter: both tokens (its own seed and the one it needs for unit 1) are fresh
    unit2 = rt.units[2]
    rt.validate_backward_prefetch_entry(unit2)


@pytest.mark.parametrize("fault,message", [
    ("wrong_owner", "reduction order"),
    ("entered", "arrived after current entry"),
    ("completed", "Completed/unvisited"),
    ("stale_token", "Stale gradient-dispatch token"),
    ("owner_not_reducing", "Invalid gradient-dispatch owner"),
])
def test_invalid_gradient_dispatch_fails_before_any_extra_gather(fault, message):
    """No dynamic fallback: a dispatch that does not fit the schedule raises, and it raises before
    another gather is issued or a generation is consumed."""
    rt, issued = _dispatch_fixture()
    owner = rt.units[3]
    if fault == "wrong_owner":
        owner = rt.units[2]
        owner.state, owner.backward_calls, owner.reductions = "GRAD_REDUCING", 1, 1
    elif fault == "entered":
        rt.units[2].backward_calls = 1
    elif fault == "completed":
        rt.units[1].reductions = 1
    elif fault == "stale_token":
        rt.units[2].generation += 1             # re-materialised behind the token's back
    elif fault == "owner_not_reducing":
        owner.state = "BWD_ACTIVE"
    generations = [u.generation for u in rt.units]
    with pytest.raises(RuntimeError, match=message):
        rt.dispatch_backward_prefetch(owner)
    assert issued == [(2, "BWD")]
    assert [u.generation for u in rt.units] == generations


def test_toy_reference_path_matches_frozen_golden_values():
    """Frozen numbers of the seeded toy stack (2 blocks, hidden 16, 4 heads, MLP 32, sequence 8,
    model seed 1234, batch seed 77): forward values, the functional oracle, and three SGD steps
    of the reference trainer.  A change of initialisation order, of the block math or of the
    trainer's loss / accumulation arithmetic shows up here even if it is self-consistent."""
    from shardtrain_b200.config import ModelConfig
    from shardtrain_b200.models.reference import build_reference_model, synthetic_batch
    from shardtrain_b200.training.reference import dense_oracle
    from shardtrain_b200.training.trainer import Trainer

    cfg = ModelConfig(layers=2, hidden_size=16, num_heads=4, mlp_hidden_size=32, seq_len=8)
    model = build_reference_model(cfg, 1234)
    x = synthetic_batch(cfg, 2, 77)
    out = model(x)
    oracle = dense_oracle(x, dict(model.named_parameters()), cfg)[-1]
    torch.testing.assert_close(out, oracle, atol=2e-6, rtol=1e-5)
    golden_row = torch.tensor([-1.31182373, 0.02675569, -0.54071665, -0.76120323, -2.77202582, 1.2404623])
    torch.testing.assert_close(out[0, 0, :6], golden_row, atol=2e-6, rtol=1e-5)
    assert out.square().mean().item() == pytest.approx(1.06242466, rel=2e-6)
    assert out.sum().item() == pytest.approx(-38.966568, rel=2e-6)
    trainer = Trainer(model, 0.05, 2)
    steps = [trainer.train_step(x) for _ in range(3)]
    golden_steps = [(1.06242466, 0.60632238, 12.5600424), (1.04437137, 0.58500424, 12.5583124),
                    (1.02754593, 0.56574057, 12.5568729)]
    for got, (loss, grad_l2, param_l2) in zip(steps, golden_steps):
        assert got.loss == pytest.approx(loss, rel=3e-6)
        assert got.gradient_l2 == pytest.approx(grad_l2, rel=3e-6)
        assert got.parameter_l2 == pytest.approx(param_l2, rel=1e-6)
    weight = dict(model.named_parameters())["1.mlp.down_proj.weight"][0, :4]
    torch.testing.assert_close(weight, torch.tensor([0.17048123, -0.1423282, 0.11148591, 0.17114937]),
                               atol=2e-7, rtol=1e-5)
