"""Communication coordinator: one submission path for every collective, tickets for their
completion, leases for buffer lifetimes, five logical streams, and the runtime event log.

Behavioural contract (reference: `src/sharded_runtime/runtime/comm.py:25-714`):

* every collective goes through `issue()`; it gets a monotonically increasing `op_id`, a per
  communicator sequence number, the leases of the buffers it touches, and (on CUDA) a
  `ready_event` recorded on its channel stream;
* a consumer calls `consume(ticket)` on *its* stream; only then is the ticket `CONSUMABLE`;
  a failing collective marks the ticket `FAILED` and later consumers raise;
* `conservative` policy chains every new collective behind the previous ticket (`PG_ORDER`
  edge, total GPU order); `stream_ordered` keeps host order only;
* buffers registered with `buffer()` must be retired exactly once, never while an issued ticket
  still references them, and none may be live at the optimizer boundary;
* every decision is recorded as a row of the event log (schema in `EVENT_DEFAULTS`), flushed to
  `runtime_events.rank{r}.jsonl` at untimed boundaries.

Three execution modes exist for a collective: `cpu` (gloo or local math), `backend_work` (NCCL:
async launch, `Work.wait()` joins the backend stream to the channel stream) and `peer_kernel`
(this package's NVLink kernels launched directly on the channel stream; ordering between GPUs is
carried by flags in peer memory, so no launch-order contract is needed).
"""

from __future__ import annotations

import json
import os
import threading
import time
from contextlib import contextmanager, nullcontext
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

CHANNELS = ("compute", "fsdp_ag", "sp_ag", "fsdp_rs", "sp_rs")
DEPENDENCY_TYPES = frozenset({"DATA_DEP", "PG_ORDER", "BUFFER_LIFETIME"})

EVENT_DEFAULTS = dict(
    op_id=None, pg_id=None, pg_seq=None, buffer_id=None, group_role=None, pg_local_seq=None,
    group_members=None, op_kind=None, producer_ticket=None, consumer_ticket=None,
    dependency_type=None, issue_stream=None, wait_stream=None, work_issued=False,
    work_wait_called=False, consumer_ready=False, last_read_complete=False,
)


@dataclass
class BufferLease:
    buffer_id: int
    tensor: object
    owner: str
    ready_event: object = None
    status: str = "ACTIVE"
    generation: int = 0

    def retire(self, stream=None) -> None:
        if self.status != "ACTIVE":
            raise RuntimeError(f"Duplicate buffer retirement {self.buffer_id}")
        if self.tensor is not None and self.tensor.is_cuda and stream is not None:
            self.tensor.record_stream(stream)
        self.tensor, self.status = None, "RETIRED"


@dataclass
class CommunicationTicket:
    op_id: int
    pg_id: str
    pg_local_seq: int
    unit_id: int | None
    phase: str
    kind: str
    work: object = None
    ready_event: object = None
    status: str = "ISSUED"
    input_leases: tuple = ()
    output_leases: tuple = ()
    group_members: tuple = ()
    issue_stream: str = "cpu"
    generation: int = 0
    group_role: str | None = None
    execution_mode: str = "cpu"
    logical_cuda_stream: int | None = None
    collective_cuda_stream: int | None = None
    api_async_op: bool | None = None
    work_returned: bool = False


def _locked(method):
    def call(self, *args, **kwargs):
        with self.submission_lock:
            return method(self, *args, **kwargs)

    call.__name__, call.__doc__ = method.__name__, method.__doc__
    return call


class StreamScope:
    """`with` block that makes one of the coordinator's streams current on its device.  Same
    effect as `torch.cuda.stream(...)` for a stream of the current device, without that
    helper's device-index lookups (several hundred scopes are entered per optimizer step)."""

    __slots__ = ("coordinator", "stream", "previous")

    def __init__(self, coordinator, stream):
        self.coordinator, self.stream, self.previous = coordinator, stream, None

    def __enter__(self):
        self.previous = self.coordinator.current_stream()
        torch.cuda.set_stream(self.stream)
        return self.stream

    def __exit__(self, *exc):
        torch.cuda.set_stream(self.previous)
        return False


class CommunicationCoordinator:
    channels = CHANNELS

    def __init__(self, device, rank=0, directory=None, *, communication_policy="conservative",
                 diagnostics_enabled=True):
        if communication_policy not in {"conservative", "stream_ordered"}:
            raise ValueError("communication_policy must be conservative or stream_ordered")
        self.communication_policy = communication_policy
        self.diagnostics_enabled = diagnostics_enabled
        self.device, self.rank = torch.device(device), rank
        # The compute stream gets the higher hardware priority: a collective kernel that is
        # already running on a side stream then cannot keep a newly launched GEMM waiting until
        # every one of its own pending thread blocks has been placed.
        self.streams = (
            {name: torch.cuda.Stream(device=self.device, priority=-1 if name == "compute" else 0)
             for name in CHANNELS}
            if self.device.type == "cuda" else {}
        )
        self.directory = Path(directory) if directory else None
        if self.directory:
            self.directory.mkdir(parents=True, exist_ok=True)
        # autograd calls into the coordinator from its own thread
        self.submission_lock = threading.RLock()
        self.tickets: list[CommunicationTicket] = []
        self.events: list[dict] = []
        self.live_buffers: dict[int, BufferLease] = {}
        self.sequence: dict[str, int] = {}
        self.expected_sequence = None
        self.next_op_id = self.next_buffer = 0
        self.step_id = -1
        self.unit_id, self.phase, self.generation, self.group_role = None, "FWD", 0, None
        self.gpu_waits: list = []
        self.pending_last_reads: list = []
        self.nccl_launch_order = None
        self.torch_build_version = str(torch.__version__)
        self._open: dict[int, CommunicationTicket] = {}     # issued, not yet consumed
        self._users: dict[int, set[int]] = {}               # buffer_id -> open op_ids
        self._by_storage: dict[int, dict[int, BufferLease]] = {}
        self._storage_of: dict[int, int] = {}
        self._group_info: dict[int, tuple] = {}
        self._log_file = None
        self._log_written = 0
        # stream_id -> the registered Stream object, for current_stream() below
        self._stream_by_id = {st.stream_id: st for st in self.streams.values()} if self.streams else {}
        self._device_index = self.device.index if self.device.type == "cuda" else None
        if self._device_index is None and self.device.type == "cuda":
            self._device_index = torch.cuda.current_device()
        if self.streams and diagnostics_enabled:
            self.event(
                "cuda_stream_registry",
                torch_build_version=self.torch_build_version,
                streams={n: {"cuda_stream": s.cuda_stream, "torch_stream_id": s.stream_id}
                         for n, s in self.streams.items()},
            )

    # ------------------------------------------------------------------ streams
    def current_stream(self):
        """The current CUDA stream of this device.  Inside a step it is almost always one of the
        runtime's own streams; those are returned from a table keyed by stream id, which skips
        the device-index normalisation and object construction of `torch.cuda.current_stream`
        (about a thousand lookups per optimizer step)."""
        probe = getattr(torch._C, "_cuda_getCurrentStream", None)
        if probe is not None and self._stream_by_id:
            known = self._stream_by_id.get(probe(self._device_index)[0])
            if known is not None:
                return known
        return torch.cuda.current_stream(self.device)

    def stream_name(self, stream=None) -> str:
        if not self.streams:
            return "cpu"
        handle = (stream or self.current_stream()).cuda_stream
        for name, registered in self.streams.items():
            if registered.cuda_stream == handle:
                return name
        return "caller"

    def stream_context(self, channel):
        return StreamScope(self, self.streams[channel]) if self.streams else nullcontext()

    def dependency(self, dependency_type, *, producer_ticket=None, consumer_ticket=None, **fields):
        if dependency_type not in DEPENDENCY_TYPES:
            raise ValueError("Unknown dependency type")
        if self.diagnostics_enabled:
            self.event("dependency_edge", dependency_type=dependency_type,
                       producer_ticket=producer_ticket, consumer_ticket=consumer_ticket, **fields)

    def wait_event(self, event, *, dependency_type, stream=None, **fields):
        if dependency_type not in DEPENDENCY_TYPES:
            raise ValueError("Unknown dependency type")
        stream = stream or self.current_stream()
        if not self.diagnostics_enabled:
            stream.wait_event(event)
            return
        waiter = self.stream_name(stream)
        self.dependency(dependency_type, wait_stream=waiter, **fields)
        if dependency_type != "PG_ORDER":
            stream.wait_event(event)
            return
        # how long the GPU really waited on a total-order edge is read later, without a sync here
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        stream.wait_event(event)
        end.record(stream)
        context = dict(fields, wait_stream=waiter, step_id=self.step_id, rank=self.rank,
                       unit_id=self.unit_id, phase=self.phase)
        self.gpu_waits.append((begin, end, context))

    def gpu_wait_timings(self):
        """Rows for finished PG_ORDER waits; call after an external synchronisation."""
        rows = [dict(ctx, dependency_type="PG_ORDER", gpu_wait_ms=b.elapsed_time(e))
                for b, e, ctx in self.gpu_waits if e.query()]
        still = []
        for event, buffer_id, generation in self.pending_last_reads:
            if event.query():
                self.event("buffer_last_read_complete", buffer_id=buffer_id, generation=generation,
                           dependency_type="BUFFER_LIFETIME", last_read_complete=True)
            else:
                still.append((event, buffer_id, generation))
        self.pending_last_reads = still
        return rows

    # ------------------------------------------------------------------ event log
    def event(self, event_type, **fields):
        if not self.diagnostics_enabled:     # the common case takes no lock
            return
        self._record_event(event_type, **fields)

    @_locked
    def _record_event(self, event_type, **fields):
        row = dict(step_id=self.step_id, rank=self.rank, unit_id=self.unit_id, phase=self.phase,
                   materialization_generation=self.generation, CPU_timestamp=time.monotonic(),
                   event_type=event_type, generation=self.generation, **EVENT_DEFAULTS)
        row["group_role"] = self.group_role
        row.update(fields)
        ticket_id = next((row[k] for k in ("op_id", "consumer_ticket", "producer_ticket")
                          if row[k] is not None), None)
        ticket = self._ticket_by_id(ticket_id)
        if ticket is not None:
            inherited = dict(
                op_id=ticket.op_id, op_kind=ticket.kind, pg_id=ticket.pg_id,
                pg_local_seq=ticket.pg_local_seq, group_members=list(ticket.group_members),
                issue_stream=ticket.issue_stream, group_role=ticket.group_role,
                execution_mode=ticket.execution_mode,
                logical_cuda_stream=ticket.logical_cuda_stream,
                collective_cuda_stream=ticket.collective_cuda_stream,
                api_async_op=ticket.api_async_op, work_returned=ticket.work_returned,
            )
            for key, value in inherited.items():
                if row.get(key) is None:
                    row[key] = value
        self.events.append(row)
        if self.streams and os.environ.get("SHARDTRAIN_NVTX") == "1":
            torch.cuda.nvtx.mark(
                f"shardtrain/{event_type}/U{row['unit_id']}/{row['phase']}/step{row['step_id']}"
                f"/op{row['op_id']}/pg{row['pg_id']}/{row['dependency_type']}"
            )

    def _ticket_by_id(self, op_id):
        if op_id is None:
            return None
        if 0 <= op_id < len(self.tickets) and self.tickets[op_id].op_id == op_id:
            return self.tickets[op_id]
        return self._open.get(op_id)

    @_locked
    def flush_diagnostics(self, *, release_events=False):
        """Append queued rows to the rank's JSONL file (no GPU synchronisation)."""
        if not self.diagnostics_enabled or self.directory is None or not self.events:
            return
        if self._log_file is None:
            path = self.directory / f"runtime_events.rank{self.rank}.jsonl"
            self._log_file = path.open("a", encoding="utf-8", buffering=1 << 20)
        for row in self.events[self._log_written:]:
            self._log_file.write(json.dumps(row, default=str) + "\n")
        self._log_written = len(self.events)
        self._log_file.flush()
        if release_events:
            self.events.clear()
            self._log_written = 0

    @_locked
    def close_diagnostics(self):
        self.flush_diagnostics()
        if self._log_file is not None:
            self._log_file.close()
            self._log_file = None

    # ------------------------------------------------------------------ leases
    @_locked
    def buffer(self, tensor, owner) -> BufferLease:
        self.next_buffer += 1
        lease = BufferLease(self.next_buffer, tensor, owner, generation=self.generation)
        self.live_buffers[lease.buffer_id] = lease
        storage = tensor.untyped_storage()
        key = storage.data_ptr()
        self._storage_of[lease.buffer_id] = key
        self._by_storage.setdefault(key, {})[lease.buffer_id] = lease
        if self.diagnostics_enabled:
            self.event("buffer_allocate", buffer_id=lease.buffer_id, owner=owner,
                       bytes=storage.nbytes(), shape=list(tensor.shape))
        return lease

    @_locked
    def retire(self, lease: BufferLease) -> None:
        if lease.status != "ACTIVE":
            raise RuntimeError(f"Duplicate buffer retirement {lease.buffer_id}")
        if self.live_buffers.get(lease.buffer_id) is not lease:
            raise RuntimeError(f"Unknown buffer lease {lease.buffer_id}")
        if self._users.get(lease.buffer_id):
            raise RuntimeError(f"Premature buffer retirement {lease.buffer_id}")
        stream = self.current_stream() if self.streams else None
        if self.diagnostics_enabled:
            if stream is not None:
                lease.ready_event = torch.cuda.Event()
                lease.ready_event.record(stream)
                self.pending_last_reads.append((lease.ready_event, lease.buffer_id, lease.generation))
            self.dependency(
                "BUFFER_LIFETIME", buffer_id=lease.buffer_id, owner=lease.owner,
                wait_stream=self.stream_name(stream), last_read_complete=stream is None,
                retirement="record_stream" if stream else "last_read_complete",
                generation=lease.generation,
            )
        lease.retire(stream)
        del self.live_buffers[lease.buffer_id]
        key = self._storage_of.pop(lease.buffer_id)
        siblings = self._by_storage[key]
        del siblings[lease.buffer_id]
        if not siblings:
            del self._by_storage[key]
        if self.diagnostics_enabled:
            self.event("buffer_retire", buffer_id=lease.buffer_id, owner=lease.owner)

    def _leases_of(self, tensors) -> tuple:
        found: dict[int, BufferLease] = {}
        for t in tensors:
            found.update(self._by_storage.get(t.untyped_storage().data_ptr(), {}))
        return tuple(found[k] for k in sorted(found))

    def _track(self, ticket):
        self._open[ticket.op_id] = ticket
        for lease in (*ticket.input_leases, *ticket.output_leases):
            self._users.setdefault(lease.buffer_id, set()).add(ticket.op_id)

    def _untrack(self, ticket):
        if self._open.pop(ticket.op_id, None) is None:
            return
        for lease in (*ticket.input_leases, *ticket.output_leases):
            users = self._users.get(lease.buffer_id)
            if users is not None:
                users.discard(ticket.op_id)
                if not users:
                    del self._users[lease.buffer_id]

    # ------------------------------------------------------------------ collectives
    def _describe_group(self, group):
        if not dist.is_initialized():
            return "local", (self.rank,), 1
        group = dist.group.WORLD if group is None else group
        cached = self._group_info.get(id(group))
        if cached is None or cached[0] is not group:
            members = tuple(dist.get_process_group_ranks(group))
            cached = (group, str(dist.get_backend(group)), members, len(members))
            self._group_info[id(group)] = cached
        return cached[1:]

    def _fail(self, ticket):
        ticket.status = "FAILED"
        self._untrack(ticket)
        if self.diagnostics_enabled:
            self.event("collective_failed", op_id=ticket.op_id)

    @_locked
    def issue(self, pg_id, kind, group, inputs, output, operation, *, channel, asynchronous,
              group_role=None, extra_outputs=(), peer_kernel=False):
        """Submit one collective.  `operation(async_op)` performs it (a torch.distributed call
        returning a Work or None, or a kernel launch when `peer_kernel`)."""
        outputs = (output, *extra_outputs)
        backend, members, group_size = self._describe_group(group)
        seq = self.sequence.get(pg_id, 0)
        if self.expected_sequence is not None:
            position = self.next_op_id
            if position >= len(self.expected_sequence) or tuple(self.expected_sequence[position]) != (pg_id, kind):
                raise RuntimeError(f"ProcessGroup order divergence at {position}: {pg_id}/{kind}")
        self.sequence[pg_id] = seq + 1
        ticket = CommunicationTicket(self.next_op_id, pg_id, seq, self.unit_id, self.phase, kind)
        self.next_op_id += 1
        ticket.group_members = members
        ticket.issue_stream, ticket.generation = channel, self.generation
        ticket.group_role = group_role or self.group_role
        if self.streams:
            ticket.logical_cuda_stream = self.streams[channel].cuda_stream
            ticket.execution_mode = "peer_kernel" if peer_kernel else "backend_work"
            ticket.api_async_op = not peer_kernel
            if peer_kernel:
                ticket.collective_cuda_stream = ticket.logical_cuda_stream
        else:
            ticket.api_async_op = asynchronous
        ticket.input_leases = self._leases_of((inputs,))
        ticket.output_leases = self._leases_of(outputs)
        previous = self.tickets[-1] if self.tickets else None
        self.tickets.append(ticket)
        self._track(ticket)
        try:
            if self.diagnostics_enabled:
                self.event(
                    "collective_issue", op_id=ticket.op_id, pg_id=pg_id, pg_seq=seq, kind=kind,
                    numel=inputs.numel(), dtype=str(inputs.dtype), op_kind=kind, pg_local_seq=seq,
                    group_members=list(members), group_role=ticket.group_role, issue_stream=channel,
                    backend=backend, input_shape=list(inputs.shape), output_shape=list(output.shape),
                    input_buffer_ids=[l.buffer_id for l in ticket.input_leases],
                    output_buffer_ids=[l.buffer_id for l in ticket.output_leases],
                    torch_build_version=self.torch_build_version,
                    extra_output_count=len(extra_outputs),
                )
            if self.streams:
                self._issue_cuda(ticket, previous, backend, group_size, inputs, outputs, operation,
                                 channel, kind, peer_kernel)
            else:
                ticket.work = operation(asynchronous)
                ticket.work_returned = ticket.work is not None
                if self.diagnostics_enabled:
                    self.event("work_issued", op_id=ticket.op_id, work_issued=ticket.work_returned,
                               issue_stream="cpu")
            if not asynchronous:
                self.consume(ticket)
            return ticket
        except BaseException:
            self._fail(ticket)
            raise

    def _issue_cuda(self, ticket, previous, backend, group_size, inputs, outputs, operation,
                    channel, kind, peer_kernel):
        ordered = self.communication_policy == "stream_ordered"
        if (ordered and backend == "nccl" and group_size > 1 and not peer_kernel
                and self.nccl_launch_order is None):
            from shardtrain_b200.distributed.nccl_ordering import require_nccl_launch_order

            self.nccl_launch_order = require_nccl_launch_order()
            if self.diagnostics_enabled:
                self.event("nccl_launch_order_contract", **self.nccl_launch_order)
        if not ordered and previous is not None:
            # total GPU order: the new collective inherits the previous one's completion
            self.consume(previous, dependency_type="PG_ORDER", consumer_ticket=ticket.op_id,
                         consumer=kind)
        produced = torch.cuda.Event()
        produced.record(self.current_stream())
        with self.stream_context(channel):
            here = self.current_stream()
            if self.diagnostics_enabled:
                self.wait_event(produced, dependency_type="DATA_DEP", consumer_ticket=ticket.op_id,
                                consumer="collective_input",
                                buffer_ids=[l.buffer_id for l in ticket.input_leases])
            else:
                here.wait_event(produced)
            if ordered and previous is not None:
                if previous.status == "FAILED":
                    raise RuntimeError(f"Failed communication {previous.op_id}")
                # host order only: no wait on previous.ready_event, or a prefetch issued earlier
                # would delay this collective's consumers
                if self.diagnostics_enabled:
                    self.event("collective_launch_order", op_id=ticket.op_id,
                               previous_op_id=previous.op_id, pg_id=ticket.pg_id,
                               pg_local_seq=ticket.pg_local_seq, issue_stream=channel,
                               ordering_scope="host_launch", gpu_completion_dependency=False)
            for tensor in (inputs, *outputs):
                if tensor.is_cuda:
                    tensor.record_stream(here)
            ticket.work = operation(ticket.api_async_op)
            ticket.work_returned = ticket.work is not None
            if self.diagnostics_enabled:
                self.event("work_issued", op_id=ticket.op_id, work_issued=ticket.work_returned,
                           issue_stream=channel)
            if ticket.work is not None:
                ticket.work.wait()  # joins the backend's stream to this channel stream
            if self.diagnostics_enabled:
                self.dependency(
                    "DATA_DEP", producer_ticket=ticket.op_id, consumer="collective_ready_event",
                    work_wait_called=ticket.work_returned,
                    completion_source="work_stream_join" if ticket.work_returned else "current_stream_event",
                    wait_stream=channel, buffer_ids=[l.buffer_id for l in ticket.output_leases],
                )
            ticket.ready_event = torch.cuda.Event()
            ticket.ready_event.record(here)

    @_locked
    def issue_kernel(self, pg_id, kind, group, launch, *, channel, after_streams=(),
                     after_events=(), numel=0, leases=(), group_role=None):
        """Submit a collective implemented by this package's own kernels.

        `launch()` enqueues the kernels; it runs with `channel`'s stream current, after that
        stream has been made to wait for the work already queued on each stream named in
        `after_streams` and for each event in `after_events`.  The ticket's `ready_event` is
        recorded behind the kernels.  Ordering between GPUs is carried by flags in peer memory,
        so neither policy adds edges here; the per-communicator sequence is still recorded.
        """
        _, members, _ = self._describe_group(group)
        seq = self.sequence.get(pg_id, 0)
        if self.expected_sequence is not None:
            position = self.next_op_id
            if position >= len(self.expected_sequence) or tuple(self.expected_sequence[position]) != (pg_id, kind):
                raise RuntimeError(f"ProcessGroup order divergence at {position}: {pg_id}/{kind}")
        self.sequence[pg_id] = seq + 1
        ticket = CommunicationTicket(self.next_op_id, pg_id, seq, self.unit_id, self.phase, kind)
        self.next_op_id += 1
        stream = self.streams[channel]
        ticket.group_members, ticket.issue_stream = members, channel
        ticket.generation, ticket.group_role = self.generation, group_role or self.group_role
        ticket.execution_mode, ticket.api_async_op = "peer_kernel", False
        ticket.logical_cuda_stream = ticket.collective_cuda_stream = stream.cuda_stream
        ticket.output_leases = tuple(leases)
        self.tickets.append(ticket)
        self._track(ticket)
        try:
            if self.diagnostics_enabled:
                self.event("collective_issue", op_id=ticket.op_id, pg_id=pg_id, pg_seq=seq, kind=kind,
                           numel=numel, dtype="torch.float32", op_kind=kind, pg_local_seq=seq,
                           group_members=list(members), group_role=ticket.group_role,
                           issue_stream=channel, backend="peer_kernel",
                           output_buffer_ids=[l.buffer_id for l in leases])
            for name in after_streams:
                produced = torch.cuda.Event()
                produced.record(self.streams[name])
                stream.wait_event(produced)
                if self.diagnostics_enabled:
                    self.dependency("DATA_DEP", consumer_ticket=ticket.op_id,
                                    consumer="collective_input", wait_stream=channel, producer_stream=name)
            for event in after_events:
                stream.wait_event(event)
            with StreamScope(self, stream):
                launch()
            if self.diagnostics_enabled:
                self.event("work_issued", op_id=ticket.op_id, work_issued=False, issue_stream=channel)
            ticket.ready_event = torch.cuda.Event()
            ticket.ready_event.record(stream)
            return ticket
        except BaseException:
            self._fail(ticket)
            raise

    @_locked
    def consume(self, ticket, *, dependency_type="DATA_DEP", consumer_ticket=None,
                consumer="collective_output"):
        """Make the calling stream (or the CPU) wait for the collective's completion."""
        if ticket.status == "FAILED":
            raise RuntimeError(f"Failed communication {ticket.op_id}")
        if dependency_type not in DEPENDENCY_TYPES:
            raise ValueError("Unknown dependency type")
        try:
            if ticket.ready_event is not None:
                if self.diagnostics_enabled:
                    self.wait_event(
                        ticket.ready_event, dependency_type=dependency_type,
                        producer_ticket=ticket.op_id, consumer_ticket=consumer_ticket,
                        consumer=consumer, producer_kind=ticket.kind, producer_unit=ticket.unit_id,
                        consumer_unit=self.unit_id, pg_id=ticket.pg_id,
                        pg_local_seq=ticket.pg_local_seq, group_members=list(ticket.group_members),
                        issue_stream=ticket.issue_stream, group_role=ticket.group_role,
                        buffer_ids=[l.buffer_id for l in ticket.output_leases],
                    )
                else:
                    self.wait_event(ticket.ready_event, dependency_type=dependency_type)
            elif ticket.work is not None:
                if self.diagnostics_enabled:
                    self.dependency(
                        dependency_type, producer_ticket=ticket.op_id,
                        consumer_ticket=consumer_ticket, consumer=consumer, wait_stream="cpu",
                        work_wait_called=True, pg_id=ticket.pg_id, pg_local_seq=ticket.pg_local_seq,
                        group_members=list(ticket.group_members), issue_stream=ticket.issue_stream,
                        group_role=ticket.group_role,
                        buffer_ids=[l.buffer_id for l in ticket.output_leases],
                    )
                ticket.work.wait()
        except BaseException:
            self._fail(ticket)
            raise
        ticket.status = "CONSUMABLE"
        self._untrack(ticket)
        ticket.work = None  # a finished Work may own the output tensors; keep metadata only
        if self.diagnostics_enabled:
            self.event(
                "collective_consumer_ready", op_id=ticket.op_id, pg_id=ticket.pg_id,
                pg_seq=ticket.pg_local_seq, pg_local_seq=ticket.pg_local_seq,
                group_members=list(ticket.group_members), consumer_ready=True,
                wait_stream=self.stream_name(), dependency_type=dependency_type,
                producer_ticket=ticket.op_id, consumer_ticket=consumer_ticket,
            )

    @_locked
    def finalize(self):
        """Consume whatever is still open, in host issue order."""
        while self._open:
            ticket = next(iter(self._open.values()))
            if ticket.status == "ISSUED":
                self.consume(ticket)
            else:
                self._untrack(ticket)

    @_locked
    def compact_completed_history(self) -> int:
        """With diagnostics off, drop finished tickets whose buffers are all retired (the newest
        ticket stays for cross-step ordering).  Returns how many were dropped."""
        if self.diagnostics_enabled or len(self.tickets) < 2:
            return 0
        newest = self.tickets[-1]

        def keep(t):
            return (t is newest or t.status != "CONSUMABLE"
                    or any(l.status != "RETIRED" for l in (*t.input_leases, *t.output_leases)))

        kept = [t for t in self.tickets if keep(t)]
        dropped = len(self.tickets) - len(kept)
        self.tickets[:] = kept
        return dropped


# ---------------------------------------------------------------------------- TP / SP group
@dataclass
class SequenceGather:
    """A sequence all-gather in flight: its input and packed output stay leased until copy-out."""

    ticket: object
    source: object
    packed: object
    source_lease: object
    packed_lease: object
    local_shape: tuple
    dim: int


def sequence_copy_out(packed, local_shape, degree, dim=1):
    """Rank-major gathered buffer [T * local] -> tensor with the T pieces concatenated on `dim`."""
    pieces = packed.view(degree, *local_shape)
    shape = list(local_shape)
    shape[dim] *= degree
    return pieces.movedim(0, dim).reshape(shape)


class RuntimeTPGroup:
    """Tensor/sequence-parallel collectives of the portable executor, split into issue and
    finish so a parameter prefetch can be submitted between the two
    (reference: `src/sharded_runtime/runtime/comm.py:731-872`)."""

    def __init__(self, group, coordinator, *, grad_group=None):
        self.process_group, self.comm = group, coordinator
        self.grad_group = grad_group if grad_group is not None else group
        live = dist.is_initialized() and group is not None
        self.degree = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.backend = str(dist.get_backend(group)) if live else "local"
        if live and grad_group is not None and grad_group is group and self.degree > 1:
            raise ValueError("Replicated-gradient SUM needs its own communicator")

    @contextmanager
    def tagged(self, role):
        saved, self.comm.group_role = self.comm.group_role, role
        try:
            yield
        finally:
            self.comm.group_role = saved

    def sequence_shard(self, x, dim=1):
        width = x.shape[dim] // self.degree
        return x.narrow(dim, self.rank * width, width).contiguous()

    def sum(self, x, *, kind="tp_allreduce", group_role=None, channel="sp_rs"):
        """Out-of-place all-reduce SUM; gradient kinds use the separate gradient communicator."""
        if self.degree == 1:
            return x
        result = x.clone()
        on_grad = kind.startswith("tp_norm") or kind.startswith("tp_grad")
        group = self.grad_group if on_grad else self.process_group
        self.comm.issue(
            "tp_grad" if on_grad else "tp", kind, group, result, result,
            lambda async_: dist.all_reduce(result, group=group, async_op=async_),
            channel=channel, asynchronous=False, group_role=group_role,
        )
        return result

    def issue_gather(self, x, dim=1) -> SequenceGather | None:
        if self.degree == 1:
            return None
        source = x.contiguous()
        packed = source.new_empty((self.degree, *source.shape))
        source_lease = self.comm.buffer(source, "sp_gather_input")
        packed_lease = self.comm.buffer(packed, "sp_gather_output")
        if self.backend == "nccl":
            def operation(async_):
                return dist.all_gather_into_tensor(packed.view(-1), source.view(-1),
                                                   group=self.process_group, async_op=async_)
        else:
            views = [packed[r] for r in range(self.degree)]

            def operation(async_):
                return dist.all_gather(views, source, group=self.process_group, async_op=async_)

        ticket = self.comm.issue("tp", "sp_ag", self.process_group, source, packed, operation,
                                 channel="sp_ag", asynchronous=True)
        return SequenceGather(ticket, source, packed, source_lease, packed_lease,
                              tuple(source.shape), dim)

    def finish_gather(self, pending: SequenceGather):
        self.comm.consume(pending.ticket, consumer="sp_gather_copy_out")
        full = pending.packed.movedim(0, pending.dim)
        shape = list(pending.local_shape)
        shape[pending.dim] *= self.degree
        gathered = full.reshape(shape)
        if gathered.data_ptr() == pending.packed.data_ptr():
            gathered = gathered.clone()
        self.comm.retire(pending.source_lease)
        self.comm.retire(pending.packed_lease)
        pending.packed = pending.source = None
        lease = self.comm.buffer(gathered, "sp_gathered_activation")
        self._activation_leases = getattr(self, "_activation_leases", {})
        self._activation_leases[gathered.data_ptr()] = lease
        return gathered

    def gather(self, x, dim=1):
        if self.degree == 1:
            return x
        return self.finish_gather(self.issue_gather(x, dim))

    def retire_activation(self, tensor):
        lease = getattr(self, "_activation_leases", {}).pop(tensor.data_ptr(), None)
        if lease is not None:
            self.comm.retire(lease)

    def reduce_scatter_sequence(self, x, dim=1):
        """SUM over the group, each rank keeping its slice of `dim`."""
        if self.degree == 1:
            return x
        width = x.shape[dim] // self.degree
        if self.backend != "nccl":
            total = x.contiguous().clone()
            self.comm.issue(
                "tp", "sp_rs_math_allreduce", self.process_group, total, total,
                lambda async_: dist.all_reduce(total, group=self.process_group, async_op=async_),
                channel="sp_rs", asynchronous=False,
            )
            return total.narrow(dim, self.rank * width, width).contiguous()
        packed = x.movedim(dim, 0).contiguous()
        out = packed.new_empty((width, *packed.shape[1:]))
        in_lease, out_lease = self.comm.buffer(packed, "sp_rs_input"), self.comm.buffer(out, "sp_rs_output")
        self.comm.issue(
            "tp", "sp_rs", self.process_group, packed, out,
            lambda async_: dist.reduce_scatter_tensor(out.view(-1), packed.view(-1),
                                                      group=self.process_group, async_op=async_),
            channel="sp_rs", asynchronous=False,
        )
        self.comm.retire(in_lease)
        self.comm.retire(out_lease)
        return out.movedim(0, dim).contiguous()
