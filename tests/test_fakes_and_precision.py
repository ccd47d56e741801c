"""Single-process checks with stand-ins, after the reference's unit tier: a dispatch-mode observer
of the GEMM operand dtypes (tests/unit/test_qwen2_gemm_precision.py:22-34), a counting fake TP
group under the shared projection (tests/unit/test_shared_projection.py:13-32), and monkeypatched
process-group calls under the distributed context (tests/unit/test_context_logging.py:25-61)."""
import logging
from collections import Counter

import pytest
import torch
from torch.utils._python_dispatch import TorchDispatchMode

from shardtrain_b200.config import ParallelConfig
from shardtrain_b200.distributed import context as context_module
from shardtrain_b200.distributed.context import DistributedContext, WorkerEnvironment
from shardtrain_b200.parallel.shared_projection import SharedProjection

GEMM_OPS = {"mm", "addmm", "bmm", "baddbmm", "linear", "matmul"}


class GemmOperands(TorchDispatchMode):
    """Records the dtypes of the tensor operands of every matrix product that reaches ATen."""

    def __init__(self):
        super().__init__()
        self.seen = Counter()

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        name = getattr(getattr(func, "overloadpacket", None), "__name__", "")
        if name in GEMM_OPS:
            self.seen[tuple(a.dtype for a in args if isinstance(a, torch.Tensor))] += 1
        return func(*args, **(kwargs or {}))


@pytest.mark.parametrize("dtype,expected", [("bf16", torch.bfloat16), ("fp32", torch.float32)])
def test_every_gemm_of_a_step_runs_in_the_compute_dtype_and_masters_stay_fp32(dtype, expected):
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    torch.manual_seed(0)
    cfg = Qwen2ModelConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2)
    model = Qwen2CausalLM(cfg)
    runtime = ShardedRuntime(device="cpu", compute_dtype=dtype).register(model)
    trainer = QwenTrainer(model, runtime, lr=1e-3, dtype=dtype, optimizer="adamw", accumulation_steps=1)
    ids = torch.randint(0, 128, (2, 16))
    with GemmOperands() as observer:
        result = trainer.train_step(ids)
    assert result.loss > 0 and observer.seen
    assert {d for operands in observer.seen for d in operands} == {expected}
    assert {p.dtype for p in model.parameters()} == {torch.float32}
    assert {p.grad.dtype for p in model.parameters()} == {torch.float32}
    state = trainer.optimizer.state
    assert all(t.dtype == torch.float32 for per in state.values() for t in per.values()
               if isinstance(t, torch.Tensor))


class CountingGroup:
    """Two sequence-parallel ranks holding the same local data, in one process: a gather is the
    local piece twice, a reduce-scatter returns this rank's slice of the two equal summands."""

    degree, rank = 2, 0

    def __init__(self):
        self.calls = Counter()

    def gather(self, x, dim):
        self.calls["gather"] += 1
        return torch.cat([x, x], dim=dim)

    def reduce_scatter_sequence(self, x):
        self.calls["reduce_scatter"] += 1
        return 2 * x[:, : x.shape[1] // 2].clone()


def test_shared_projection_gathers_once_per_direction_and_saves_only_the_local_shard():
    torch.manual_seed(1)
    x = torch.randn(2, 4, 8, requires_grad=True)
    weights = [torch.randn(6, 8, requires_grad=True) for _ in range(3)]
    group = CountingGroup()
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(tuple(t.shape)) or t, lambda t: t):
        outs = SharedProjection.apply(x, group, *weights)
    assert group.calls == {"gather": 1}                      # one gather feeds three projections
    assert (2, 8, 8) not in saved and (2, 4, 8) in saved     # the gathered input is not kept
    grads = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, grads)
    assert group.calls == {"gather": 2, "reduce_scatter": 1}  # one re-gather, one reduce-scatter
    full = torch.cat([x.detach(), x.detach()], dim=1)
    for w, g in zip(weights, grads):
        torch.testing.assert_close(w.grad, g.reshape(-1, 6).t() @ full.reshape(-1, 8))
    dx = sum(g @ w.detach() for g, w in zip(grads, weights))
    torch.testing.assert_close(x.grad, 2 * dx[:, :4])
    with pytest.raises(RuntimeError, match="trainable"):
        SharedProjection.apply(x, group, weights[0], torch.randn(6, 8))


def test_context_creates_groups_in_topology_order_and_tears_down_without_a_barrier(monkeypatch):
    """Rank 1 of F2 x T2 on a faked gloo world: every communicator of the creation order is
    created (creation is collective), only this rank's are kept, close callbacks run first, the
    kept groups are destroyed in reverse and the default group last, a failing step is recorded
    while the later ones still run, and nothing ever calls a barrier."""
    log = []
    dist = context_module.dist
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", "29999")
    monkeypatch.setattr(dist, "is_initialized", lambda: False)
    monkeypatch.setattr(dist, "init_process_group", lambda **kw: log.append(("init", kw["backend"], kw["rank"])))
    monkeypatch.setattr(dist, "new_group", lambda ranks, **kw: log.append(("new", tuple(ranks))) or tuple(ranks))

    def destroy(group=None):
        log.append(("destroy", group))
        if group == (0, 1):
            raise RuntimeError("injected teardown failure")

    monkeypatch.setattr(dist, "destroy_process_group", destroy)
    monkeypatch.setattr(dist, "barrier", lambda *a, **k: pytest.fail("cleanup must not wait for peers"))
    parallel = ParallelConfig(fsdp_degree=2, tp_degree=2, sp_enabled=False, device="cpu", backend="gloo")
    context = DistributedContext(parallel, WorkerEnvironment(1, 1, 4, True), 30, logging.getLogger("t"))
    created = [entry[1] for entry in log if entry[0] == "new"]
    assert created == [tuple(members) for _, members in context.topology.creation_order]
    assert log[0] == ("init", "gloo", 1)
    mine = [g for g in created if 1 in g]
    assert context.tp_group == (0, 1) and context.fsdp_group == (1, 3) and context.sp_group is context.tp_group
    context.add_close_callback(lambda: log.append(("callback",)))
    mark = len(log)
    context.close()
    context.close()                                            # idempotent
    teardown = log[mark:]
    assert teardown[0] == ("callback",)
    assert [e[1] for e in teardown[1:]] == list(reversed(mine)) + [None]
    # (0, 1) is this rank's TP communicator and, as a second communicator, its TP gradient group
    assert len(context.cleanup_errors) == mine.count((0, 1)) == 2
    assert all("injected" in text for text in context.cleanup_errors)
    assert context.tp_group is None and context.fsdp_group is None
    with pytest.raises(RuntimeError, match="closed"):
        context.add_close_callback(lambda: None)
