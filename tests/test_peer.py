"""Single-member behaviour of the peer-memory layer (the multi-member paths need several GPUs and
are exercised by tests/workers/qwen_worker.py under torchrun)."""
import pytest
import torch

from shardtrain_b200.distributed.peer import CHANNEL_SLOTS, METRIC_WIDTH, PeerMemory


def test_single_member_group_uses_plain_tensors_and_no_kernels():
    peer = PeerMemory(None, "cpu", ops=None)
    assert peer.degree == 1 and peer.rank == 0 and peer.flags is None and peer.inbox is None
    buf = peer.alloc(1000)
    assert buf.nbytes == 1024 and buf.ptrs == [buf.local_ptr] and buf.owner.numel() == 1024
    assert not buf.owner.any()
    peer.barrier("fsdp_rs")                      # no-op: would need ops otherwise
    assert peer.epochs["fsdp_rs"] == 0
    peer.close()


def test_small_all_reduce_of_one_member_is_the_identity():
    peer = PeerMemory(None, "cpu", ops=None)
    values = torch.tensor([3.0, -1.5, 7.0], dtype=torch.float64)
    out = peer.all_reduce_small(values, min_mask=0b010)
    assert torch.equal(out, values) and out.data_ptr() != values.data_ptr()
    with pytest.raises(ValueError):
        peer.all_reduce_small(torch.zeros(3))                               # not float64
    with pytest.raises(ValueError):
        peer.all_reduce_small(torch.zeros(METRIC_WIDTH + 1, dtype=torch.float64))


def test_every_barrier_channel_has_its_own_flag_slot():
    slots = list(CHANNEL_SLOTS.values())
    assert len(set(slots)) == len(slots) and max(slots) < 4096 // (8 * 4)


class _FakeOps:
    """Records the order of the CUDA-IPC calls `PeerMemory` makes (no GPU involved)."""

    def __init__(self):
        self.calls, self._next = [], 1000

    def peer_alloc(self, nbytes):
        self._next += 4096
        self.calls.append(("alloc", self._next))
        return self._next

    def ipc_handle(self, ptr):
        return torch.full((64,), ptr % 251, dtype=torch.uint8)

    def ipc_open(self, handle):
        self._next += 4096
        self.calls.append(("open", self._next))
        return self._next

    def ipc_close(self, ptr):
        self.calls.append(("close", ptr))

    def peer_free(self, ptr):
        self.calls.append(("free", ptr))

    def device_synchronize(self):
        self.calls.append(("sync", None))


@pytest.fixture
def two_member_group(monkeypatch):
    """A fake two-member process group: rank 0, whose peer always answers like rank 0 does."""
    import torch.distributed as dist

    state = {"fail": False, "log": []}

    def all_gather_object(out, obj, group=None):
        if state["fail"]:
            raise RuntimeError("peer is gone")
        state["log"].append(obj)
        for i in range(len(out)):
            out[i] = obj

    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(dist, "get_rank", lambda group=None: 0)
    monkeypatch.setattr(dist, "all_gather_object", all_gather_object)
    return state


def test_close_frees_exported_buffers_only_after_every_member_reported_idle(two_member_group):
    ops = _FakeOps()
    peer = PeerMemory(object(), "cpu", ops, wait_seconds=0.5)
    assert peer.wait_us == 500_000
    peer.alloc(1 << 20)
    ops.calls.clear()
    two_member_group["log"].clear()
    assert peer.close() is True
    kinds = [k for k, _ in ops.calls]
    # device idle, then imports closed, then (after the host handshake) exported buffers freed
    assert kinds[0] == "sync"
    assert kinds.index("free") > max(i for i, k in enumerate(kinds) if k == "close")
    assert kinds.count("close") == 3 and kinds.count("free") == 3      # flags, inbox, buffer
    assert two_member_group["log"] == [("idle", 0)]
    assert peer.close() is False                                        # idempotent


def test_close_after_a_failure_leaks_instead_of_freeing_under_a_reader(two_member_group):
    ops = _FakeOps()
    peer = PeerMemory(object(), "cpu", ops)
    peer.alloc(4096)
    ops.calls.clear()
    assert peer.close(failed=True) is False
    assert ops.calls == []                      # nothing unmapped, nothing freed, no handshake


def test_close_leaks_when_the_handshake_cannot_complete(two_member_group):
    ops = _FakeOps()
    peer = PeerMemory(object(), "cpu", ops)
    peer.alloc(4096)
    ops.calls.clear()
    two_member_group["fail"] = True
    assert peer.close() is False
    assert not any(kind == "free" for kind, _ in ops.calls)


def test_wait_budget_is_clamped_to_seconds():
    assert PeerMemory(None, "cpu", None, wait_seconds=300).wait_us == 10_000_000
    with pytest.raises(ValueError):
        PeerMemory(None, "cpu", None, wait_seconds=0)
