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
