import pytest
import torch

from shardtrain_b200.runtime.layout import (ArenaPlan, ParameterSpec, ShardedParameter, copy_out,
                                            offsets, pack_gradients, padding_ranges, segment_table,
                                            shard_of)


def specs_for(shapes, degree):
    return [ParameterSpec.create(f"p{i}", 0, torch.empty(s), s, "column", degree)
            for i, s in enumerate(shapes)]


@pytest.mark.parametrize("degree", [1, 2, 4, 8])
def test_pack_gather_roundtrip_with_odd_sizes(degree):
    torch.manual_seed(degree)
    shapes = [(3, 5), (7,), (2, 2, 3), (1,), (8, 8)]
    specs = specs_for(shapes, degree)
    tensors = [torch.randn(s) for s in shapes]
    starts, slot = offsets(specs)
    assert slot == sum(-(-t.numel() // degree) for t in tensors)
    # every rank's slot, then the rank-major packed gather buffer
    storage = torch.zeros(degree * slot)
    for rank in range(degree):
        for t, spec, start in zip(tensors, specs, starts):
            storage[rank * slot + start: rank * slot + start + spec.fsdp_shard_numel] = shard_of(t, spec, rank)
    out = copy_out(storage, specs, degree)
    for t, spec in zip(tensors, specs):
        assert torch.equal(out[spec.param_id], t)
        assert spec.padding_numel == degree * spec.fsdp_shard_numel - t.numel()
        assert sum(spec.valid_len(r) for r in range(degree)) == t.numel()
    # destination-major gradient packing is the inverse placement, padding exactly zero
    packed = pack_gradients(tensors, specs, degree).view(degree, slot)
    for rank in range(degree):
        for t, spec, start in zip(tensors, specs, starts):
            keep = spec.valid_len(rank)
            q = spec.fsdp_shard_numel
            assert torch.equal(packed[rank, start:start + keep], t.reshape(-1)[rank * q: rank * q + keep])
            assert packed[rank, start + keep:start + q].abs().sum() == 0


def test_pack_rejects_wrong_shape():
    specs = specs_for([(2, 3)], 2)
    with pytest.raises(RuntimeError, match="Invalid full gradient"):
        pack_gradients([torch.zeros(3, 2)], specs, 2)


def test_arena_plan_alignment_and_tables():
    specs = specs_for([(5,), (3, 3), (2,)], 2)
    plan = ArenaPlan()
    handles = []
    for spec in specs:
        h = ShardedParameter(spec, None)
        h.arena_offset = plan.add(spec)
        handles.append(h)
    assert [h.arena_offset % 4 for h in handles] == [0, 0, 0]
    assert plan.unit_ranges[0] == (0, plan.total)
    assert padding_ranges(handles, 1) == [(handles[0].arena_offset + 2, handles[0].arena_offset + 3),
                                          (handles[1].arena_offset + 4, handles[1].arena_offset + 5)]
    table = segment_table(handles, {"p0": 0, "p1": 8, "p2": 24}, {"p0"})
    assert table.shape == (3, 5) and table[0].tolist() == [0, 3, 5, 0, 1]


def test_arena_offsets_keep_bf16_shadows_16_byte_aligned():
    """Shard offsets are multiples of 8 elements: 32 bytes in the FP32 arenas and 16 bytes in
    the bf16 shadow arena that mirrors them (vector loads of the gather kernel)."""
    plan = ArenaPlan()
    for spec in specs_for([(5,), (3, 3), (2,), (17, 3)], 2):
        assert plan.add(spec) % 8 == 0
    assert plan.padded_total() % 8 == 0


def test_reduce_table_marks_tp_replicated_parameters():
    """Flag bit 1 of a reduce table row tells the reduce-scatter kernel to sum that parameter
    over the whole F x T mesh; gather tables never carry it."""
    split = ParameterSpec.create("w", 0, torch.empty(4, 6), (8, 6), "column", 2)
    repl = ParameterSpec.create("norm", 0, torch.empty(6), (6,), "replicated", 2)
    handles = []
    plan = ArenaPlan()
    for spec in (split, repl):
        h = ShardedParameter(spec, None)
        h.arena_offset = plan.add(spec)
        handles.append(h)
    offsets_ = {"w": 0, "norm": 24}
    reduce = segment_table(handles, offsets_, set(), mark_replicated=True)
    assert reduce[:, 4].tolist() == [0, 2]
    gather = segment_table(handles, offsets_, {"norm"})
    assert gather[:, 4].tolist() == [0, 1]
    assert reduce[1].tolist()[:4] == [handles[1].arena_offset, 3, 6, 24]
