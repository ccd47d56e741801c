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
