"""Parameter materialisation and gradient reduction for one FSDP group.

Two implementations share the lease / ticket protocol of the coordinator:

* `Materializer` -- portable.  Packed rank-major all-gather through `torch.distributed`
  (`all_gather_into_tensor` on NCCL, list `all_gather` on gloo), copy-out into independent FP32
  full parameters, and destination-major packed reduce-scatter (all-reduce + slice on gloo) with
  the 1/F average and the TP SUM of replicated parameters.  It is the CPU path and the in-repo
  NCCL baseline (behaviour of `src/sharded_runtime/runtime/materializer.py:31-271`).
* `PeerMaterializer` -- sm_100a.  The gather is one kernel that pulls every peer's FP32 shards
  over NVLink and lands compute-dtype (bf16) full parameters in a leased unit buffer; the
  reduction is one kernel that pulls this rank's slice of every peer's full FP32 gradient,
  averages, accumulates into the persistent gradient arena and, on the last micro-step,
  applies AdamW in the same pass.  Cross-GPU ordering is a flag barrier in peer memory.

Both commit reduced gradients straight into the runtime's gradient arena.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from shardtrain_b200.runtime.layout import copy_out, offsets, pack_gradients


@dataclass
class MaterializationLease:
    unit_id: int
    step_id: int
    phase: str
    generation: int
    ag_storage: object = None
    full_param_storages: dict = field(default_factory=dict)
    ag_ticket: object = None
    copy_out_ready_event: object = None
    fullparam_last_consumer_event: object = None
    weights: dict = field(default_factory=dict)   # name -> full parameter tensor
    extras: dict = field(default_factory=dict)    # executor-specific views (fused layouts)


def _group_shape(group):
    live = dist.is_initialized() and group is not None
    if not live:
        return 1, 0, "local"
    return dist.get_world_size(group), dist.get_rank(group), str(dist.get_backend(group))


class Materializer:
    kind = "portable"

    def __init__(self, group, coordinator):
        self.group, self.comm = group, coordinator
        self.degree, self.rank, self.backend = _group_shape(group)

    # ------------------------------------------------------------------ parameters
    @torch.no_grad()
    def issue(self, unit, phase) -> MaterializationLease:
        runtime = unit.runtime
        specs = [h.spec for h in unit.handles]
        starts, slot_len = offsets(specs)
        anchor = unit.handles[0].local_shard
        with self.comm.stream_context("fsdp_ag"):
            # shards depend on the optimizer's writes, not on activations queued on compute
            if self.comm.streams:
                runtime.wait_parameter_shards_ready()
            storage = anchor.new_empty(self.degree * slot_len)
            lease = MaterializationLease(unit.unit_id, runtime.step_id, phase, unit.generation,
                                         self.comm.buffer(storage, "fsdp_ag"))
            mine = storage.narrow(0, self.rank * slot_len, slot_len)
            for handle, start in zip(unit.handles, starts):
                mine.narrow(0, start, handle.spec.fsdp_shard_numel).copy_(handle.local_shard)
            if self.degree > 1:
                if self.backend == "nccl":
                    def operation(async_):
                        return dist.all_gather_into_tensor(storage, mine, group=self.group,
                                                           async_op=async_)
                else:
                    slots = [storage.narrow(0, r * slot_len, slot_len) for r in range(self.degree)]

                    def operation(async_):
                        return dist.all_gather(slots, mine, group=self.group, async_op=async_)

                lease.ag_ticket = self.comm.issue(
                    "fsdp", "fsdp_ag", self.group, mine, storage, operation, channel="fsdp_ag",
                    asynchronous=runtime.asynchronous, group_role="parameter_materialization",
                )
            elif self.comm.streams:
                lease.copy_out_ready_event = torch.cuda.Event()
                lease.copy_out_ready_event.record(torch.cuda.current_stream(anchor.device))
        return lease

    def _await_gather(self, unit, lease):
        if lease.ag_ticket:
            self.comm.consume(lease.ag_ticket, consumer=f"copy_out/U{unit.unit_id}")
        elif lease.copy_out_ready_event is not None:
            self.comm.wait_event(lease.copy_out_ready_event, dependency_type="DATA_DEP",
                                 consumer=f"copy_out/U{unit.unit_id}",
                                 buffer_id=lease.ag_storage.buffer_id)
        if self.comm.diagnostics_enabled:
            self.comm.event("copy_out_start", unit_id=unit.unit_id,
                            producer_ticket=lease.ag_ticket.op_id if lease.ag_ticket else None,
                            buffer_id=lease.ag_storage.buffer_id,
                            issue_stream=self.comm.stream_name())

    def finish(self, unit):
        lease = unit.lease
        if lease.extras.pop("carried", False):
            # kept from the previous micro-step of the same optimizer step: nothing to do
            return tuple(lease.weights[h.spec.param_id] for h in unit.handles)
        if lease.full_param_storages:
            raise RuntimeError(f"Duplicate copy-out U{unit.unit_id}")
        self._await_gather(unit, lease)
        weights = copy_out(lease.ag_storage.tensor, [h.spec for h in unit.handles], self.degree)
        for name, weight in weights.items():
            lease.full_param_storages[name] = self.comm.buffer(weight, "full_parameter")
        lease.weights = weights
        if self.comm.streams:
            lease.copy_out_ready_event = torch.cuda.Event()
            lease.copy_out_ready_event.record(self.comm.current_stream())
        self.comm.event("copy_out_ready", unit_id=unit.unit_id)
        # nothing keeps the packed buffer alive past copy-out
        self.comm.retire(lease.ag_storage)
        lease.ag_storage = None
        return tuple(weights[h.spec.param_id] for h in unit.handles)

    # ------------------------------------------------------------------ gradients
    def _issue_bucket(self, unit, grads, specs, bucket):
        group = getattr(unit.runtime, "fsdp_grad_group", None) or self.group
        packed = pack_gradients(grads, specs, self.degree)
        source = self.comm.buffer(packed, f"fsdp_{bucket}_rs_input")
        starts, slot_len = offsets(specs)
        output = packed.new_empty(slot_len)
        ticket = ready = None
        if self.degree == 1:
            output.copy_(packed)
            if self.comm.streams:
                here = self.comm.current_stream()
                packed.record_stream(here)
                output.record_stream(here)
                ready = torch.cuda.Event()
                ready.record(here)
        elif self.backend != "nccl":
            ticket = self.comm.issue(
                "fsdp_grad", "fsdp_rs_math_allreduce", group, packed, packed,
                lambda async_: dist.all_reduce(packed, group=group, async_op=async_),
                channel="fsdp_rs", asynchronous=unit.runtime.async_grad_rs,
                group_role=f"{bucket}_gradient_bucket",
            )
        else:
            ticket = self.comm.issue(
                "fsdp_grad", "fsdp_rs", group, packed, output,
                lambda async_: dist.reduce_scatter_tensor(output, packed, group=group, async_op=async_),
                channel="fsdp_rs", asynchronous=unit.runtime.async_grad_rs,
                group_role=f"{bucket}_gradient_bucket",
            )
        if self.comm.diagnostics_enabled:
            self.comm.event("gradient_bucket_issued", bucket=bucket,
                            parameters=[s.param_id for s in specs],
                            producer_ticket=ticket.op_id if ticket else None,
                            source_buffer_id=source.buffer_id, output_numel=slot_len)
        return dict(output=output, packed=packed, source=source, starts=starts, ticket=ticket,
                    ready=ready)

    def _consume_bucket(self, state, bucket):
        output, packed, ticket = state["output"], state["packed"], state["ticket"]
        if ticket is not None:
            self.comm.consume(ticket, consumer=f"{bucket}_gradient_bucket")
        elif state["ready"] is not None:
            self.comm.wait_event(state["ready"], dependency_type="DATA_DEP",
                                 consumer=f"{bucket}_gradient_bucket",
                                 buffer_id=state["source"].buffer_id)
        if self.degree > 1 and self.backend != "nccl":
            output.copy_(packed.narrow(0, self.rank * output.numel(), output.numel()))
        output.div_(self.degree)  # the one FSDP average of every parameter
        if self.comm.streams:
            output.record_stream(self.comm.current_stream())
        self.comm.retire(state["source"])
        self.comm.event("gradient_bucket_consumed", bucket=bucket,
                        producer_ticket=ticket.op_id if ticket else None)
        return output, state["starts"]

    def reduce(self, unit, grads):
        """Reduce-scatter the unit's full gradients and commit the shards to the arena."""
        runtime = unit.runtime
        specs = [h.spec for h in unit.handles]
        if len(grads) != len(specs) or any(g is None for g in grads):
            raise RuntimeError(f"Missing full parameter gradient U{unit.unit_id}")
        split = runtime.communication_policy == "stream_ordered" and runtime.async_grad_rs
        small = [i for i, s in enumerate(specs)
                 if split and s.tp_grad_reduce == "sum" and len(s.tp_local_shape) == 1]
        large = [i for i in range(len(specs)) if i not in small]
        # the small replicated vectors go first so their TP SUM (own communicator) can start
        # while the large bucket is still on the wire
        pending = {}
        for bucket, members in (("norm", small), ("main", large)):
            if members:
                pending[bucket] = self._issue_bucket(unit, [grads[i] for i in members],
                                                     [specs[i] for i in members], bucket)
        if getattr(runtime, "gradient_dispatch_prefetch", False):
            runtime.dispatch_backward_prefetch(unit)
        tp = runtime.tp
        for bucket, members, channel in (("norm", small, "compute"), ("main", large, None)):
            if not members:
                continue
            context = self.comm.stream_context(channel) if channel else _null()
            with context:
                output, starts = self._consume_bucket(pending[bucket], bucket)
                for i, start in zip(members, starts):
                    spec = specs[i]
                    shard_grad = output.narrow(0, start, spec.fsdp_shard_numel)
                    if spec.tp_grad_reduce == "sum":
                        if not runtime.sp:
                            shard_grad = shard_grad / tp.degree
                        shard_grad = tp.sum(shard_grad, kind="tp_norm_allreduce",
                                            group_role="norm_gradient_bucket" if bucket == "norm" else None,
                                            channel="compute" if bucket == "norm" else "sp_rs")
                    runtime.commit_gradient(unit.handles[i], shard_grad)
                if bucket == "norm" and self.comm.streams:
                    done = torch.cuda.Event()
                    done.record(self.comm.current_stream())
                    self.comm.wait_event(done, dependency_type="DATA_DEP",
                                         stream=self.comm.streams["fsdp_rs"] if runtime.async_grad_rs else None,
                                         consumer=f"autograd_norm_shard/U{unit.unit_id}",
                                         producer_unit=unit.unit_id)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class PeerMaterializer:
    """sm_100a materialiser: gather+cast and reduce-scatter(+AdamW) kernels over peer memory.

    `plans[unit_id]` (built at registration by the fused executor) carries, per unit, the segment
    tables of the two kernels, the unit's persistent compute-dtype buffers with every parameter
    view precomputed, and the one-element FP32 tokens used as autograd edges.  The buffers are
    allocated once (180 GB of HBM makes a per-unit bf16 copy cheap); "resharding" a unit ends the
    *validity* of its buffer -- lease, generation and step checks are unchanged -- so the next use
    must gather again, but no allocator traffic or view construction happens inside a step.
    """

    kind = "peer"

    def __init__(self, group, coordinator, peer_memory):
        self.group, self.comm, self.peer = group, coordinator, peer_memory
        self.degree, self.rank, self.backend = _group_shape(group)
        self.plans: dict[int, object] = {}
        self.ops = None

    def bind(self, ops, arenas):
        """`arenas`: object with param/grad/exp_avg/exp_avg_sq flat tensors and peer pointers."""
        self.ops, self.arenas = ops, arenas

    @torch.no_grad()
    def issue(self, unit, phase) -> MaterializationLease:
        runtime = unit.runtime
        plan = self.plans[unit.unit_id]
        comm = self.comm
        lease = MaterializationLease(unit.unit_id, runtime.step_id, phase, unit.generation)
        lease.ag_storage = comm.buffer(plan.full_bf16, "fsdp_ag")
        lease.extras["full_bf16"], lease.extras["full_fp32"] = plan.full_bf16, plan.full_fp32
        ptrs = self.arenas.param_peer_ptrs
        # a decoder layer's forward may pull q|k|v and gate|up inside its GEMMs: the gather
        # kernel then lands only the other parameters
        pull = self.arenas.pulls_in_gemm(unit, phase)
        table = plan.gather_table_rest if pull else plan.gather_table
        lease.extras["pull_in_gemm"] = pull

        def launch():
            # the shards depend on the optimizer's writes (and on every peer having finished
            # its own), never on activations queued on the compute stream
            runtime.wait_parameter_shards_ready()
            if table.numel():     # empty when the unit's buffer aliases the shadow
                shadows = [] if runtime.wire_dtype == "fp32" else self.arenas.shadow_peer_ptrs
                self.ops.gather_params(ptrs, table, plan.full_bf16, plan.full_fp32, shadows)

        # a buffer may be re-gathered only after its last reader on the compute stream
        after = (plan.last_reader,) if plan.last_reader is not None else ()
        lease.ag_ticket = comm.issue_kernel(
            "fsdp", "fsdp_ag_partial" if pull else "fsdp_ag_cast", self.group, launch,
            channel="fsdp_ag", after_events=after, numel=plan.shard_numel, leases=(lease.ag_storage,),
            group_role="parameter_materialization")
        return lease

    def finish(self, unit):
        lease = unit.lease
        plan = self.plans[unit.unit_id]
        if lease.extras.pop("carried", False):
            return plan.tokens
        if lease.weights:
            raise RuntimeError(f"Duplicate copy-out U{unit.unit_id}")
        comm = self.comm
        # A tied embedding unit is entered by the embedding lookup, which reads rows from the
        # owners' FP32 shards and needs nothing of the gathered table; the LM head at the END of
        # the forward is the table's first reader.  The wait for the (large) gather moves there,
        # so the decoder layers run while it is still crossing the link; the lookup only needs
        # the peers' shards to be final, which the barrier before the gather established.
        defer = (getattr(unit, "tied", False) and lease.phase == "FWD" and self.degree > 1
                 and comm.streams and getattr(self.arenas, "shards_clean_event", None) is not None)
        if defer:
            unit.runtime.wait_parameter_shards_ready()
            comm.wait_event(self.arenas.shards_clean_event, dependency_type="DATA_DEP",
                            consumer=f"embedding_lookup/U{unit.unit_id}")
            lease.extras["deferred_gather"] = lease.ag_ticket
        else:
            comm.consume(lease.ag_ticket, consumer=f"copy_out/U{unit.unit_id}")
        plan = self.plans[unit.unit_id]
        if comm.diagnostics_enabled:
            comm.event("copy_out_start", unit_id=unit.unit_id, producer_ticket=lease.ag_ticket.op_id,
                       buffer_id=lease.ag_storage.buffer_id, issue_stream=comm.stream_name())
        # the gather kernel already landed every parameter in its final place and dtype: the
        # "copy-out" is handing out the precomputed views
        lease.weights = plan.weights
        lease.full_param_storages["bf16"] = lease.ag_storage
        lease.ag_storage = None
        lease.copy_out_ready_event = None if defer else lease.ag_ticket.ready_event
        comm.event("copy_out_ready", unit_id=unit.unit_id, deferred=bool(defer))
        # The autograd edges of this executor carry one-element FP32 tokens, not the bf16
        # weights: autograd would cast an FP32 weight gradient to the dtype of a bf16 edge.  The
        # kernels read the weights from the lease and write gradients into the unit's slot.
        return plan.tokens

    def await_deferred(self, unit):
        """Make the calling stream wait for a gather whose wait `finish` left to the first real
        reader of the gathered parameters (no-op when nothing was deferred)."""
        lease = unit.lease
        ticket = lease.extras.pop("deferred_gather", None) if lease is not None else None
        if ticket is not None:
            self.comm.consume(ticket, consumer=f"copy_out/U{unit.unit_id}")
            lease.copy_out_ready_event = ticket.ready_event

    def released(self, unit, event):
        """Called when the unit's full parameters are given up; `event` marks the last reader."""
        self.await_deferred(unit)      # a gather nobody waited for must not outlive its buffer
        self.plans[unit.unit_id].last_reader = event

    def reduce(self, unit, grads):
        """The fused backward already wrote every full gradient into the unit's slot; `grads`
        are the token gradients that made autograd schedule this reduction."""
        runtime = unit.runtime
        plan = self.plans[unit.unit_id]
        if len(grads) != len(unit.handles) or any(g is None for g in grads):
            raise RuntimeError(f"Missing full parameter gradient U{unit.unit_id}")
        slot = runtime.fused.grad_slot(unit)          # peer-visible buffer holding the gradients
        first = runtime.first_commit(unit)
        fuse_adamw = runtime.fused_optimizer_armed(unit)
        arenas = self.arenas

        # TP axis of the reduction: the slot table lists the whole mesh; TP-replicated
        # parameters are summed over it (each TP rank saw its own sequence slice)
        # with SP every TP rank saw its own sequence slice (sum); without SP all TP ranks hold the
        # same gradient of a replicated parameter (average)
        replicated_scale = 1.0 / self.degree if runtime.sp else 1.0 / (self.degree * arenas.tp_degree)
        tp = (arenas.tp_degree, arenas.tp_rank, replicated_scale)

        # NVLS: the switch adds the members' slots (only when the ring got multicast addresses)
        multicast = slot.multicast_ptr if getattr(arenas, "nvls_active", False) else 0

        def launch():
            arenas.reduce_peer.barrier("fsdp_rs")     # no-op for a single member
            if fuse_adamw:
                hp = runtime.fused_optimizer_args()
                self.ops.reduce_scatter_adamw(
                    slot.peer_ptrs, self.rank, plan.reduce_table, arenas.grad, arenas.param,
                    arenas.exp_avg, arenas.exp_avg_sq, 1.0 / self.degree, not first, *hp,
                    arenas.check_flags, *tp, arenas.shadow, multicast)
            else:
                self.ops.reduce_scatter(slot.peer_ptrs, self.rank, plan.reduce_table, arenas.grad,
                                        1.0 / self.degree, not first, arenas.check_flags, *tp,
                                        multicast)

        comm = self.comm
        ticket = comm.issue_kernel(
            "fsdp_grad", "fsdp_rs_accumulate_adamw" if fuse_adamw else "fsdp_rs_accumulate",
            self.group, launch, channel="fsdp_rs", after_streams=("compute",),
            numel=plan.grad_numel, group_role="main_gradient_bucket")
        if not runtime.async_grad_rs:
            comm.consume(ticket, consumer="main_gradient_bucket")
        if comm.diagnostics_enabled:
            comm.event("gradient_bucket_issued", bucket="main",
                       parameters=[h.spec.param_id for h in unit.handles],
                       producer_ticket=ticket.op_id, output_numel=plan.shard_numel)
        runtime.fused.grad_slot_issued(unit, slot, ticket)
        if getattr(runtime, "gradient_dispatch_prefetch", False):
            runtime.dispatch_backward_prefetch(unit)
        for handle in unit.handles:
            runtime.mark_committed(handle, ticket)
        if fuse_adamw:
            runtime.note_fused_update(unit)
