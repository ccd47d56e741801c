"""The communication volume model against the figures the reference published for Qwen2.5-1.5B
(reports/fsdp_interview_sections/04_communication_volume.md:84-95 and
reports/fsdp4_vs_hybrid_2x2_native_4gpu.md:76): counts and ideal-ring bytes per rank per step."""
import pytest

from shardtrain_b200.utils.comm_volume import predict, qwen_units

QWEN15B = dict(hidden_size=1536, mlp_hidden_size=8960, num_heads=12, num_key_value_heads=2, layers=28,
               vocab_size=151936, seq_len=512, tie_word_embeddings=True)


def test_unit_plan_adds_up_to_the_published_parameter_count():
    units = qwen_units(QWEN15B, 1)
    assert len(units) == 30
    assert sum(u.split + u.replicated for u in units) == 1_543_714_304
    assert units[1].split + units[1].replicated == 46_797_824
    # a TP-local layer in FP32 is the 93 601 792-byte all-gather the reference timed with nccl-tests
    half = qwen_units(QWEN15B, 2)[1]
    assert 4 * (half.split + half.replicated) == 93_601_792


def test_hybrid_f2t2_sp_matches_the_published_inventory():
    got = predict(QWEN15B, fsdp=2, tp=2, sp=True, local_batch=4, accumulation=2)
    roles = got["roles"]
    assert (roles["fsdp_param_allgather"]["count"], roles["fsdp_param_allgather"]["bytes"]) == (116, 6_175_201_280)
    assert (roles["fsdp_grad_reduce_scatter"]["count"], roles["fsdp_grad_reduce_scatter"]["bytes"]) == (116, 3_554_351_104)
    assert (roles["sp_activation_allgather"]["count"], roles["sp_activation_allgather"]["bytes"]) == (336, 1_056_964_608)
    assert (roles["sp_activation_reduce_scatter"]["count"], roles["sp_activation_reduce_scatter"]["bytes"]) == (224, 1_056_964_608)
    assert (roles["tp_norm_grad_allreduce"]["count"], roles["tp_norm_grad_allreduce"]["bytes"]) == (114, 350_208)
    assert (roles["tp_replicated_grad_allreduce"]["count"], roles["tp_replicated_grad_allreduce"]["bytes"]) == (2, 933_494_784)
    assert got["collectives"] == 908
    assert got["bytes"] == pytest.approx(12.777e9, rel=1e-4)


def test_f4t1_matches_the_published_total():
    got = predict(QWEN15B, fsdp=4, tp=1, sp=False, local_batch=2, accumulation=2)
    assert got["bytes"] == pytest.approx(26.387e9, rel=1e-4)
    assert got["roles"]["fsdp_grad_reduce_scatter"]["count"] == 60
    assert set(got["roles"]) == {"fsdp_param_allgather", "fsdp_grad_reduce_scatter"}


def test_peer_wire_halves_the_matrix_gather_and_needs_no_tensor_parallel_allreduce():
    ref = predict(QWEN15B, fsdp=8, tp=1, sp=False, local_batch=1, accumulation=2)
    peer = predict(QWEN15B, fsdp=8, tp=1, sp=False, local_batch=1, accumulation=2, wire="peer")
    ratio = peer["roles"]["fsdp_param_allgather"]["bytes"] / ref["roles"]["fsdp_param_allgather"]["bytes"]
    assert 0.5 < ratio < 0.5001                       # bf16 matrices, FP32 vectors
    assert peer["roles"]["fsdp_grad_reduce_scatter"]["bytes"] == ref["roles"]["fsdp_grad_reduce_scatter"]["bytes"]
    hybrid = predict(QWEN15B, fsdp=4, tp=2, sp=True, local_batch=2, accumulation=2, wire="peer")
    assert not any("allreduce" in role for role in hybrid["roles"])
    assert hybrid["roles"]["fsdp_grad_reduce_scatter"]["count"] == 60
    # per layer backward at F8T1: the bytes each GPU takes in (gradients in FP32, parameters in bf16)
    layer = qwen_units(QWEN15B, 1)[1]
    numel = layer.split + layer.replicated
    assert round(7 / 8 * 4 * numel / 1e6) == 164 and round(7 / 8 * 2 * numel / 1e6) == 82
