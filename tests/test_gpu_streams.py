"""Stream and lifetime behaviour of the coordinator on a real GPU, with fake Work objects and short
device-side delays (about a millisecond each; nothing here waits on another GPU).  The rules are
those of the reference's CUDA suite (tests/cuda/test_runtime_cuda.py:19-351): `conservative`
chains every collective behind the previous one's completion, `stream_ordered` keeps host order
only, a delayed parameter gather never holds up a sequence reduce-scatter or its consumer, and the
unit's reduction runs on the reduce-scatter stream exactly when gradient reduction is asynchronous."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
DELAY_CYCLES = 3_000_000       # ~1.5 ms at 1.9 GHz


class NoWork:
    """A "collective" that completes on the stream it was issued on (nothing to wait for)."""

    def wait(self):
        return None


def coordinator(policy):
    from shardtrain_b200.runtime.comm import CommunicationCoordinator

    return CommunicationCoordinator(torch.device("cuda", 0), communication_policy=policy)


def timed_collective(comm, pg, kind, channel, *, delay):
    """Issue a fake collective whose device work is `delay` cycles of sleep followed by a write;
    returns (ticket, start event, end event) with the events recorded on the channel stream."""
    src, dst = torch.ones(4, device="cuda"), torch.zeros(4, device="cuda")
    marks = {}

    def operation(async_op):
        here = torch.cuda.current_stream()
        marks["begin"] = torch.cuda.Event(enable_timing=True)
        marks["begin"].record(here)
        if delay:
            torch.cuda._sleep(delay)
        dst.copy_(src)
        marks["end"] = torch.cuda.Event(enable_timing=True)
        marks["end"].record(here)
        return NoWork()

    ticket = comm.issue(pg, kind, None, src, dst, operation, channel=channel, asynchronous=True)
    return ticket, marks["begin"], marks["end"], dst


def test_five_distinct_streams_and_stream_names():
    comm = coordinator("stream_ordered")
    assert sorted(comm.streams) == ["compute", "fsdp_ag", "fsdp_rs", "sp_ag", "sp_rs"]
    assert len({s.cuda_stream for s in comm.streams.values()}) == 5
    with comm.stream_context("sp_rs"):
        assert comm.stream_name() == "sp_rs"


def test_conservative_policy_chains_collectives_and_stream_ordered_does_not():
    origin = torch.cuda.Event(enable_timing=True)
    results = {}
    for policy in ("conservative", "stream_ordered"):
        comm = coordinator(policy)
        torch.cuda.synchronize()
        origin.record()
        slow = timed_collective(comm, "fsdp", "fake_param_gather", "fsdp_ag", delay=DELAY_CYCLES)
        fast = timed_collective(comm, "tp", "fake_seq_reduce_scatter", "sp_rs", delay=0)
        comm.consume(fast[0])
        comm.consume(slow[0])
        torch.cuda.synchronize()
        results[policy] = (origin.elapsed_time(slow[2]), origin.elapsed_time(fast[1]))
        assert slow[3].sum().item() == 4 and fast[3].sum().item() == 4
        edges = [e for e in comm.events if e["event_type"] == "dependency_edge"
                 and e["dependency_type"] == "PG_ORDER"]
        assert bool(edges) == (policy == "conservative")
    slow_end, fast_begin = results["conservative"]
    assert fast_begin >= slow_end - 0.05          # total order on the GPU
    slow_end, fast_begin = results["stream_ordered"]
    assert fast_begin < slow_end - 0.3            # the reduce-scatter did not wait for the gather


def test_delayed_next_unit_gather_blocks_neither_the_reduce_scatter_nor_its_consumer():
    """Host order: gather (slow) first, reduce-scatter second.  The compute stream consumes the
    reduce-scatter and finishes long before the gather does; consuming the gather later still
    sees its data (host launch order is not a completion wait)."""
    comm = coordinator("stream_ordered")
    compute = comm.streams["compute"]
    # the first use of a kernel loads its module on the host (tens of milliseconds): run every op
    # of the timed part once, so that what is timed below is device ordering, not the host
    warm = timed_collective(comm, "tp", "fake_seq_reduce_scatter", "sp_rs", delay=1000)
    with torch.cuda.stream(compute):
        comm.consume(warm[0], consumer="warm_up")
        assert ((warm[3] * 2).sum().item(), (warm[3] + 1).sum().item()) == (8, 8)
    torch.cuda.synchronize()
    origin = torch.cuda.Event(enable_timing=True)
    origin.record()
    # ~30 ms of device sleep: far longer than any hiccup of the host between the launches below
    gather = timed_collective(comm, "fsdp", "fake_param_gather", "fsdp_ag", delay=20 * DELAY_CYCLES)
    scatter = timed_collective(comm, "tp", "fake_seq_reduce_scatter", "sp_rs", delay=0)
    with torch.cuda.stream(compute):
        comm.consume(scatter[0], consumer="row_linear_output")
        used = scatter[3] * 2
        consumed = torch.cuda.Event(enable_timing=True)
        consumed.record(compute)
        assert gather[0].status == "ISSUED"        # still open on the host side
        comm.consume(gather[0], consumer="copy_out")
        late = gather[3] + 1
    torch.cuda.synchronize()
    assert used.sum().item() == 8 and late.sum().item() == 8
    assert origin.elapsed_time(consumed) < origin.elapsed_time(gather[2]) - 1.0
    waits = [e for e in comm.events if e["event_type"] == "dependency_edge"
             and e.get("consumer") == "row_linear_output"]
    assert waits and all(e["dependency_type"] == "DATA_DEP" for e in waits)


def test_premature_retirement_is_refused_until_the_collective_was_consumed():
    comm = coordinator("stream_ordered")
    dst = torch.zeros(4, device="cuda")
    lease = comm.buffer(dst, "fsdp_ag")
    ticket = comm.issue("fsdp", "fake", None, torch.ones(4, device="cuda"), dst,
                        lambda a: NoWork(), channel="fsdp_ag", asynchronous=True)
    with pytest.raises(RuntimeError, match="Premature buffer retirement"):
        comm.retire(lease)
    comm.consume(ticket)
    comm.retire(lease)
    assert not comm.live_buffers


@pytest.mark.parametrize("async_rs", [False, True])
def test_unit_reduction_runs_on_the_reduce_scatter_stream_iff_asynchronous(async_rs):
    """Portable executor on CUDA, degree 1: the bridge node of every unit lives on `fsdp_rs` when
    `async_grad_rs` is on (so the reduction is not serialised behind compute) and on `compute`
    otherwise; results match the dense model either way."""
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.qwen2_trainer import QwenTrainer

    torch.manual_seed(0)
    cfg = Qwen2ModelConfig(vocab_size=256, hidden_size=64, intermediate_size=128,
                           num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2)
    dense = Qwen2CausalLM(cfg).cuda()
    model = copy.deepcopy(dense)
    rt = ShardedRuntime(device="cuda:0", reshard_after_forward=True, forward_prefetch=True,
                        backward_prefetch=True, async_grad_rs=async_rs,
                        communication_policy="stream_ordered", communication_backend="nccl",
                        compute_dtype="fp32").register(model)
    tr = QwenTrainer(model, rt, lr=0.05, dtype="fp32", optimizer="sgd")
    ids = torch.randint(0, 256, (2, 32), device="cuda")
    got = tr.train_step(ids)
    want = dense(ids, labels=ids).loss
    assert got.loss == pytest.approx(want.item(), rel=2e-5)
    ready = [e for e in rt.comm.events if e["event_type"] == "unit_grads_ready"]
    assert len(ready) == 5
    streams = {e.get("issue_stream") or e.get("current_stream") for e in ready}
    assert streams == ({"fsdp_rs"} if async_rs else {"compute"}), streams
    assert not rt.comm.live_buffers
