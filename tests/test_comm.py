"""Coordinator contract with fake Work objects (no process group needed)."""
import pytest
import torch

from shardtrain_b200.runtime.comm import CommunicationCoordinator


class DelayedWork:
    """`wait()` performs the data movement, so a consumer that never waited sees stale data."""

    def __init__(self, action):
        self.action, self.waited = action, False

    def wait(self):
        if not self.waited:
            self.action()
            self.waited = True


class FailingWork:
    def wait(self):
        raise RuntimeError("injected collective failure")


def test_consumer_sees_data_only_after_consume_and_leases_guard_retirement():
    comm = CommunicationCoordinator("cpu")
    src, dst = torch.ones(4), torch.zeros(4)
    lease = comm.buffer(dst, "out")
    ticket = comm.issue("fsdp", "fake_ag", None, src, dst, lambda a: DelayedWork(lambda: dst.copy_(src)),
                        channel="fsdp_ag", asynchronous=True)
    assert ticket.status == "ISSUED" and dst.sum() == 0
    with pytest.raises(RuntimeError, match="Premature buffer retirement"):
        comm.retire(lease)
    comm.consume(ticket)
    assert ticket.status == "CONSUMABLE" and dst.sum() == 4 and ticket.work is None
    comm.retire(lease)
    with pytest.raises(RuntimeError, match="Duplicate buffer retirement"):
        comm.retire(lease)
    assert not comm.live_buffers


def test_out_of_order_consumption_and_finalize():
    comm = CommunicationCoordinator("cpu")
    done = []
    tickets = [comm.issue("tp", f"k{i}", None, torch.zeros(1), torch.zeros(1),
                          lambda a, i=i: DelayedWork(lambda: done.append(i)),
                          channel="sp_ag", asynchronous=True) for i in range(3)]
    comm.consume(tickets[2])
    assert done == [2]
    comm.finalize()
    assert done == [2, 0, 1] and all(t.status == "CONSUMABLE" for t in tickets)
    assert [t.pg_local_seq for t in tickets] == [0, 1, 2]


def test_failed_collective_poisons_later_consumers():
    comm = CommunicationCoordinator("cpu")
    t = comm.issue("fsdp", "bad", None, torch.zeros(1), torch.zeros(1), lambda a: FailingWork(),
                   channel="fsdp_rs", asynchronous=True)
    with pytest.raises(RuntimeError, match="injected"):
        comm.consume(t)
    assert t.status == "FAILED"
    with pytest.raises(RuntimeError, match=f"Failed communication {t.op_id}"):
        comm.consume(t)
    kinds = [e["event_type"] for e in comm.events]
    assert "collective_failed" in kinds


def test_expected_sequence_divergence_is_detected():
    comm = CommunicationCoordinator("cpu")
    comm.expected_sequence = [("fsdp", "a"), ("tp", "b")]
    comm.issue("fsdp", "a", None, torch.zeros(1), torch.zeros(1), lambda a: None, channel="fsdp_ag",
               asynchronous=False)
    with pytest.raises(RuntimeError, match="order divergence at 1"):
        comm.issue("fsdp", "c", None, torch.zeros(1), torch.zeros(1), lambda a: None,
                   channel="fsdp_ag", asynchronous=False)


def test_event_log_schema_and_flush(tmp_path):
    comm = CommunicationCoordinator("cpu", rank=3, directory=tmp_path)
    comm.unit_id, comm.phase, comm.step_id = 2, "BWD", 7
    comm.issue("fsdp", "x", None, torch.zeros(2), torch.zeros(2), lambda a: None, channel="fsdp_ag",
               asynchronous=False)
    row = next(e for e in comm.events if e["event_type"] == "collective_issue")
    for key in ("step_id", "rank", "unit_id", "phase", "materialization_generation", "CPU_timestamp",
                "op_id", "pg_id", "pg_seq", "buffer_id", "group_role", "dependency_type",
                "issue_stream", "wait_stream"):
        assert key in row
    assert (row["rank"], row["unit_id"], row["phase"], row["step_id"]) == (3, 2, "BWD", 7)
    comm.flush_diagnostics()
    lines = (tmp_path / "runtime_events.rank3.jsonl").read_text().splitlines()
    assert len(lines) == len(comm.events)
    comm.close_diagnostics()
    quiet = CommunicationCoordinator("cpu", diagnostics_enabled=False)
    quiet.issue("fsdp", "x", None, torch.zeros(2), torch.zeros(2), lambda a: None, channel="fsdp_ag",
                asynchronous=False)
    assert not quiet.events and quiet.tickets[0].status == "CONSUMABLE"
    assert quiet.compact_completed_history() == 0


@pytest.mark.parametrize("degree,rank", [(1, 0), (2, 0), (2, 1)])
@pytest.mark.parametrize("sp", [False, True])
def test_norm_bucket_sum_runs_while_the_main_reduction_is_still_pending(monkeypatch, degree, rank, sp):
    """Two gradient buckets with delayed fake Work (the data only moves in `wait()`): the small
    replicated-vector bucket is issued first and its TP SUM happens while the main bucket's
    reduce-scatter has not been waited for; values follow (sum over F) / F, then the T-way SUM
    (divided by T first when the activations were replicated, i.e. without SP); padding of the
    committed shards stays zero; nothing stays leased."""
    from types import SimpleNamespace

    from shardtrain_b200.runtime.layout import ParameterSpec
    from shardtrain_b200.runtime.materializer import Materializer

    grads = [torch.arange(1.0, 6.0), torch.arange(1.0, 13.0).reshape(4, 3),
             torch.arange(1.0, 4.0), torch.arange(1.0, 19.0).reshape(6, 3)]
    layouts = ["replicated", "column", "column", "replicated"]
    specs = [ParameterSpec.create(f"p{i}", 0, g, g.shape, lay, degree)
             for i, (g, lay) in enumerate(zip(grads, layouts))]
    comm = CommunicationCoordinator("cpu", communication_policy="stream_ordered")
    works, order, commits = [], [], {}

    class PeerContribution:
        """The other FSDP member holds 3 x this rank's gradient: the sum is 4 g."""

        def __init__(self, output, packed):
            self.output, self.packed, self.waited = output, packed, False
            works.append(self)

        def wait(self):
            if not self.waited:
                lo = rank * self.output.numel()
                self.output.copy_(self.packed[lo:lo + self.output.numel()] * 4)
                self.waited = True
                order.append(("rs_waited", len([w for w in works if w.waited])))

    def fake_reduce_scatter(output, packed, *, group=None, async_op=False):
        assert async_op
        return PeerContribution(output, packed)

    def tp_sum(gradient, *, kind, group_role=None, channel="sp_rs"):
        assert kind == "tp_norm_allreduce"
        order.append(("tp_sum", group_role, channel))
        if group_role == "norm_gradient_bucket" and degree > 1:
            assert works[0].waited and not works[1].waited
        return gradient.clone() * 6          # the other TP member holds 5 x this one's value

    monkeypatch.setattr(torch.distributed, "reduce_scatter_tensor", fake_reduce_scatter)
    runtime = SimpleNamespace(
        fsdp_grad_group=None, communication_policy="stream_ordered", async_grad_rs=True, sp=sp,
        tp=SimpleNamespace(degree=2, sum=tp_sum), gradient_dispatch_prefetch=False,
        commit_gradient=lambda handle, shard: commits.__setitem__(handle.spec.param_id, shard.clone()))
    unit = SimpleNamespace(runtime=runtime, unit_id=0,
                           handles=[SimpleNamespace(spec=s) for s in specs])
    mat = Materializer(None, comm)
    mat.degree, mat.rank, mat.backend = degree, rank, "nccl"    # a simulated 2-rank NCCL world
    mat.reduce(unit, grads)

    for g, spec in zip(grads, specs):
        full = g.clone() if degree == 1 else (g + 3 * g) / 2
        if spec.tp_grad_reduce == "sum":
            full = (full if sp else full / 2) * 6
        want = torch.zeros(spec.fsdp_shard_numel)
        keep = spec.valid_len(rank)
        want[:keep] = full.flatten()[rank * spec.fsdp_shard_numel: rank * spec.fsdp_shard_numel + keep]
        torch.testing.assert_close(commits[spec.param_id], want, atol=0, rtol=0)
    sums = [o for o in order if o[0] == "tp_sum"]
    assert sums == [("tp_sum", "norm_gradient_bucket", "compute"), ("tp_sum", None, "sp_rs")]
    assert not comm.live_buffers and all(w.waited for w in works)
    issued = [e["bucket"] for e in comm.events if e["event_type"] == "gradient_bucket_issued"]
    assert issued == ["norm", "main"]
    roles = [t.group_role for t in comm.tickets]
    assert roles == (["norm_gradient_bucket", "main_gradient_bucket"] if degree > 1 else [])


def test_reduce_rejects_a_missing_gradient():
    from types import SimpleNamespace

    from shardtrain_b200.runtime.layout import ParameterSpec
    from shardtrain_b200.runtime.materializer import Materializer

    g = torch.arange(1.0, 6.0)
    spec = ParameterSpec.create("p", 0, g, g.shape, "replicated", 1)
    comm = CommunicationCoordinator("cpu")
    unit = SimpleNamespace(runtime=SimpleNamespace(), unit_id=3, handles=[SimpleNamespace(spec=spec)])
    with pytest.raises(RuntimeError, match="Missing full parameter gradient U3"):
        Materializer(None, comm).reduce(unit, [None])
