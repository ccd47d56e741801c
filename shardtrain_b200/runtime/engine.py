"""`ShardedRuntime`: persistent FP32 shard leaves, per-unit materialisation state machine,
prefetch scheduling and step boundaries.

Behaviour kept from the reference engine (`src/sharded_runtime/runtime/engine.py:20-709`):

* unit states `SHARDED -> FWD_MATERIALIZING -> FWD_ACTIVE -> RESHARDED | FWD_RETAINED ->
  BWD_MATERIALIZING -> BWD_ACTIVE -> GRAD_REDUCING -> GRAD_READY -> SHARDED`, `FAILED` on error;
  each unit runs forward, backward and reduction exactly once per micro-step; every
  materialisation bumps the unit's `generation` and backward weight reads must come from the
  current step and generation;
* who issues the next parameter gather: at unit entry (plain prefetch), inside the consumer that
  owns the boundary handle when sequence-parallel collectives are stream-ordered (deferred
  prefetch), or from the previous unit's gradient dispatch with validated tokens
  (`gradient_dispatch_prefetch`);
* the optimizer may hold only the shard leaves and may step only after `finalize_backward`;
  its post-step hook publishes the shard-writer event that the next gather waits for.

What differs by design: all shard leaves (and their `.grad`) are views into two flat arenas, the
reduced gradients are committed into the gradient arena by the unit's reduction itself, the model
forward is driven by the runtime (`model_forward`) instead of module hooks, and on sm_100a the
materialiser / executor pair is `PeerMaterializer` + `FusedExecutor` (hand-written kernels).
"""

from __future__ import annotations

from contextlib import contextmanager

import torch
import torch.distributed as dist
from torch import nn

from shardtrain_b200.runtime.bridge import PreBackward, UnitMaterialize
from shardtrain_b200.runtime.comm import CommunicationCoordinator, RuntimeTPGroup
from shardtrain_b200.runtime.layout import ArenaPlan, ParameterSpec, ShardedParameter, padding_ranges
from shardtrain_b200.runtime.materializer import Materializer

MATERIALIZED_WAITING = {"RESHARDED", "FWD_RETAINED", "FWD_MATERIALIZING", "BWD_MATERIALIZING"}

# The life of a unit inside one micro-step, as a table: state -> states it may be entered from.
# ("SHARDED" enters FWD_ACTIVE directly when the lease was carried over from the previous
# micro-step; FAILED is entered from anywhere by `ShardedRuntime.fail`.)
# One edge is a quirk kept from the reference: with deferred sequence-parallel prefetch the tied LM
# head (second consumer of unit 0's boundary handle) triggers "the next unit's forward gather"
# once more at the end of the forward, so unit 1 goes RESHARDED -> FWD_MATERIALIZING and enters
# its backward on that lease.
ENTERED_FROM = {
    "FWD_MATERIALIZING": {"SHARDED", "RESHARDED"},
    "FWD_ACTIVE": {"FWD_MATERIALIZING", "SHARDED"},
    "RESHARDED": {"FWD_ACTIVE"},
    "FWD_RETAINED": {"FWD_ACTIVE"},
    "BWD_MATERIALIZING": {"RESHARDED"},
    "BWD_ACTIVE": {"BWD_MATERIALIZING", "FWD_RETAINED", "FWD_MATERIALIZING"},
    "GRAD_REDUCING": {"BWD_ACTIVE"},
    "GRAD_READY": {"GRAD_REDUCING"},
}
DIRECTION = {"FWD": +1, "BWD": -1}      # which neighbour a phase prefetches


class UnitState:
    """One FSDP unit: a group of parameters gathered, used, re-gathered and reduced together.

    The unit is a small state machine (`ENTERED_FROM`) plus three counters that pin "exactly once
    per micro-step" for forward, backward and reduction.  Who issues the neighbour's gather is
    decided in one place, `_gather_neighbour`, from the runtime's prefetch switches."""

    tied = False

    def __init__(self, runtime, unit_id, block):
        self.runtime, self.unit_id, self.block = runtime, unit_id, block
        self.handles: list[ShardedParameter] = []
        self.generation = 0
        self.state = "SHARDED"
        self.lease = None
        self.forward_calls = self.backward_calls = self.reductions = 0
        self.forward_prefetch_handle = self.backward_prefetch_handle = None
        self.forward_weights: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ bookkeeping
    def annotate(self, phase):
        comm = self.runtime.comm
        comm.unit_id, comm.phase, comm.generation = self.unit_id, phase, self.generation

    def handle(self, name) -> ShardedParameter:
        return self.runtime.registry[name]

    def _enter(self, state):
        if self.state not in ENTERED_FROM[state]:
            raise RuntimeError(f"Illegal unit transition U{self.unit_id}: {self.state} -> {state}")
        self.state = state

    def _once(self, counter, what):
        """`counter` (forward_calls, backward_calls, reductions) goes 0 -> 1 exactly once."""
        if not self.runtime.active or getattr(self, counter):
            raise RuntimeError(f"{what} U{self.unit_id}")
        setattr(self, counter, 1)

    # ------------------------------------------------------------------ materialisation
    def issue(self, phase):
        if self.lease is not None:
            raise RuntimeError(f"Duplicate materialization U{self.unit_id} {phase}")
        self.generation += 1
        self.annotate(phase)
        self._enter(f"{phase}_MATERIALIZING")
        self.lease = self.runtime.materializer.issue(self, phase)
        self.runtime.comm.event("materialize_issue")

    def release(self):
        if self.lease is None:
            raise RuntimeError(f"Missing lease U{self.unit_id}")
        comm, lease = self.runtime.comm, self.lease
        if comm.streams:
            lease.fullparam_last_consumer_event = torch.cuda.Event()
            lease.fullparam_last_consumer_event.record(comm.current_stream())
        notify = getattr(self.runtime.materializer, "released", None)
        if notify is not None:
            notify(self, lease.fullparam_last_consumer_event)
        for storage in lease.full_param_storages.values():
            comm.retire(storage)
        lease.full_param_storages.clear()
        lease.weights = {}
        self.lease = None
        comm.event("fullparams_retired", unit_id=self.unit_id)

    def weight(self, name):
        """Full parameter for a backward consumer, from the current step and generation only."""
        lease = self.lease
        if self.state != "BWD_ACTIVE" or lease is None:
            raise RuntimeError(f"Stale/early weight consumer {name} U{self.unit_id} {self.state}")
        if (lease.step_id, lease.generation) != (self.runtime.step_id, self.generation):
            raise RuntimeError(f"Stale generation {name}")
        return lease.weights[name]

    # ------------------------------------------------------------------ who gathers the neighbour
    def _gather_neighbour(self, phase, *, at, handle=None):
        """Issue the gather of the unit this phase reaches next, if this is the place that owns
        the decision.  `at` names the caller:

        * "entry"  - the unit was just entered (`pre_forward` / `pre_backward`);
        * "input"  - a consumer has issued its sequence collective (`prefetch_after_input`).

        Plain prefetch decides at entry.  When sequence-parallel collectives are stream-ordered
        the decision moves behind the consumer that owns the boundary handle ("input"), except
        for an asynchronous backward, which keeps entry (or the gradient-dispatch tokens) as its
        single scheduling source."""
        runtime = self.runtime
        enabled = runtime.forward_prefetch if phase == "FWD" else runtime.backward_prefetch
        target = self.unit_id + DIRECTION[phase]
        if not enabled or not 0 <= target < len(runtime.units):
            return
        deferred = runtime.defer_sp_prefetch and not (phase == "BWD" and runtime.async_grad_rs)
        if at == "input":
            boundary = self.forward_prefetch_handle if phase == "FWD" else self.backward_prefetch_handle
            if not deferred or handle is not boundary:
                return
            self.annotate(phase)
            runtime.comm.event("prefetch_boundary", param_id=handle.spec.param_id, target_unit=target)
        else:
            if deferred:
                return
            if phase == "BWD":
                runtime.comm.event("prefetch_boundary", target_unit=target,
                                   scheduling_boundary="backward_unit_entry")
        runtime.prefetch(target, phase)
        if at == "input" or phase == "BWD":
            self.annotate(phase)       # (a forward entry leaves the log annotated with the target)

    def prefetch_after_input(self, handle, phase):
        """Deferred prefetch: called by a consumer after it issued its sequence collective."""
        self._gather_neighbour(phase, at="input", handle=handle)

    # ------------------------------------------------------------------ forward
    def pre_forward(self, *_):
        runtime = self.runtime
        self._once("forward_calls", "Forward outside begin_step or repeated Unit")
        if self.lease is None:
            self.issue("FWD")
        self.annotate("FWD")
        # the bridge node lives on the reduce-scatter stream when gradients reduce asynchronously,
        # so its backward (the reduction) is not serialised behind compute
        channel = "fsdp_rs" if runtime.async_grad_rs else "compute"
        with runtime.comm.stream_context(channel):
            weights = UnitMaterialize.apply(self, *(h.local_shard for h in self.handles))
        if isinstance(weights, torch.Tensor):
            weights = (weights,)
        self.forward_weights = {h.spec.param_id: w for h, w in zip(self.handles, weights)}
        self._enter("FWD_ACTIVE")
        runtime.comm.event("unit_forward")
        self._gather_neighbour("FWD", at="entry")

    def forward_weight(self, name, *, tied_second_use=False):
        """Autograd-connected full parameter for a forward consumer (one use per parameter)."""
        if self.state != "FWD_ACTIVE" or name not in self.forward_weights:
            raise RuntimeError("Consumer has no current forward materialization")
        self.handle(name).mark_forward(tied_second_use=tied_second_use)
        return self.forward_weights[name]

    def post_forward(self, output):
        runtime = self.runtime
        self.forward_weights = {}
        self.annotate("FWD")
        last = self.unit_id == len(runtime.units) - 1
        if runtime.reshard_after_forward and not last and not runtime.retain_parameters:
            self.release()
            self._enter("RESHARDED")
        else:
            self._enter("FWD_RETAINED")
        runtime.comm.event(self.state)
        return PreBackward.apply(output, self)

    # ------------------------------------------------------------------ backward
    def pre_backward(self):
        runtime = self.runtime
        if not runtime.active or self.backward_calls:
            raise RuntimeError(f"Repeated/invalid backward U{self.unit_id}; retain_graph unsupported")
        dispatch = runtime.gradient_dispatch_prefetch
        if dispatch:
            runtime.validate_backward_prefetch_entry(self)
        self.backward_calls += 1
        if self.lease is None:
            self.issue("BWD")
        self.annotate("BWD")
        if not self.lease.weights:
            runtime.materializer.finish(self)
        self._enter("BWD_ACTIVE")
        runtime.comm.event("unit_pre_backward")
        if dispatch:
            runtime.backward_prefetch_entered(self)
        else:
            self._gather_neighbour("BWD", at="entry")

    def reduce(self, grads):
        if self.reductions or self.state != "BWD_ACTIVE":
            raise RuntimeError(f"Duplicate/early gradient RS U{self.unit_id} {self.state}")
        self.reductions += 1
        self.annotate("BWD")
        self._enter("GRAD_REDUCING")
        comm = self.runtime.comm
        if comm.diagnostics_enabled:
            # the stream this node runs on: autograd replays the stream of the bridge's forward
            comm.event("unit_grads_ready", parameters=[h.spec.param_id for h in self.handles],
                       issue_stream=comm.stream_name())
        self.runtime.materializer.reduce(self, grads)
        if self.runtime.retain_parameters and not self.runtime.last_microstep:
            # parameters do not change between micro-steps: keep the gathered copy
            self.runtime.retained_leases[self.unit_id] = self.lease
            self.lease = None
        else:
            self.release()
        self._enter("GRAD_READY")


class TiedEmbeddingUnit(UnitState):
    """Unit 0 of a tied model: one shard, used by the embedding first and the LM head last.

    Its full parameter stays materialised from the embedding to the end of backward; the two
    adjoints meet on the single bridge output, so there is one reduction
    (`src/sharded_runtime/runtime/qwen2_adapter.py:27-49`).
    """

    tied = True

    def pre_forward(self, *args):
        runtime = self.runtime
        materializer = runtime.materializer
        if (self.lease is None and runtime.forward_prefetch and not runtime.defer_sp_prefetch
                and len(runtime.units) > 1 and getattr(materializer, "kind", "") == "peer"
                and materializer.degree > 1):
            # On the sm_100a path the embedding lookup reads the shards and the gathered table is
            # first read by the LM head at the end of the forward, while the first layer needs
            # its weights at once: its (much smaller) gather goes first on the gather stream.
            runtime.prefetch(1, "FWD")
            self.annotate("FWD")
        super().pre_forward(*args)

    def embedding_complete(self):
        self.annotate("FWD")
        if self.runtime.forward_prefetch and len(self.runtime.units) > 1:
            self.runtime.prefetch(1, "FWD")
            self.annotate("FWD")

    def head_complete(self, output):
        if self.handles[0].forward_uses != 2:
            raise RuntimeError("Tied weight must have exactly embedding and head forward uses")
        self.forward_weights = {}
        self.annotate("FWD")
        self._enter("FWD_RETAINED")
        self.runtime.comm.event("tied_weight_retained", unit_id=self.unit_id)
        return PreBackward.apply(output, self)


class ShardedRuntime:
    def __init__(self, *, device="cpu", reshard_after_forward=True, forward_prefetch=False,
                 backward_prefetch=False, async_grad_rs=False, communication_policy="conservative",
                 directory=None, diagnostics_enabled=True, communication_backend="auto",
                 retain_parameters=False, compute_dtype=None, device_wait_seconds=2.0,
                 wire_dtype="bf16", fused_allgather="auto", fused_seq_gather=False, nvls="off",
                 cuda_graphs=True):
        self.device = torch.device(device)
        self.reshard_after_forward = reshard_after_forward
        self.forward_prefetch, self.backward_prefetch = forward_prefetch, backward_prefetch
        self.async_grad_rs = async_grad_rs
        self.asynchronous = forward_prefetch or backward_prefetch or async_grad_rs
        self.communication_policy = communication_policy
        self.communication_backend = communication_backend
        self.retain_parameters = retain_parameters
        # dtype of the GEMM operands the trainer will ask for ("fp32", "fp16", "bf16"; None =
        # not stated).  Only bf16 (or unstated) runs may be given to the sm_100a executor.
        if compute_dtype not in (None, "fp32", "fp16", "bf16"):
            raise ValueError("compute_dtype must be fp32, fp16 or bf16")
        self.requested_dtype = compute_dtype
        # what the sm_100a parameter gather moves over NVLink: the bf16 shadow of the shards
        # (same bits as gather-then-cast, half the bytes) or the fp32 shards themselves
        if wire_dtype not in ("bf16", "fp32"):
            raise ValueError("wire_dtype must be bf16 or fp32")
        self.wire_dtype = wire_dtype
        # sm_100a, FSDP degree > 1: whether a decoder layer's forward pulls q|k|v and gate|up
        # from the owners' shards inside the consuming GEMMs instead of gathering them first
        if fused_allgather not in ("auto", "on", "off"):
            raise ValueError("fused_allgather must be auto, on or off")
        self.fused_allgather = fused_allgather
        # sm_100a, sequence parallel: the GEMM that consumes a sequence all-gather pulls the
        # peers' slices itself (one kernel) instead of running after a gather kernel.  Off by
        # default: on two B200s the pulling GEMM was 7-9 % slower per training step than the
        # gather kernel followed by the plain GEMM (its producer has to poll arrival flags)
        self.fused_seq_gather = bool(fused_seq_gather)
        # sm_100a, FSDP-only meshes: a decoder layer's forward / backward launch sequence is
        # captured into a CUDA graph the second time it is called with identical arguments and
        # replayed from then on (activations then live in buffers the executor owns)
        self.cuda_graphs = bool(cuda_graphs)
        # sm_100a, FSDP-only meshes: reduce gradients inside the NVSwitch (`multimem.ld_reduce`
        # over multicast-bound gradient slots).  "auto": when the fabric grants multicast, else
        # plain peer loads; "off": never bind memory to a multicast object.
        if nvls not in ("auto", "off"):
            raise ValueError("nvls must be auto or off")
        self.nvls = nvls
        # time budget of every device-side wait on a peer (seconds; clamped by PeerMemory)
        self.device_wait_seconds = float(device_wait_seconds)
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.comm = CommunicationCoordinator(self.device, rank, directory,
                                             communication_policy=communication_policy,
                                             diagnostics_enabled=diagnostics_enabled)
        self.units: list[UnitState] = []
        self.registry: dict[str, ShardedParameter] = {}
        self.identities: dict[str, tuple[int, int]] = {}
        self.step_id = -1
        self.active = self.optimizer_ready = self.failed = False
        self.sp = False
        self.defer_sp_prefetch = False
        self.parameter_shards_ready_event = None
        self.parameter_shards_version = 0
        self.backward_prefetch_tokens: dict = {}
        self.backward_entry_expected = self.backward_dispatch_expected = None
        self.plan = ArenaPlan()
        self.param_arena = self.grad_arena = None
        self.grad_epoch = 0
        self.last_microstep = True
        self.retained_leases: dict[int, object] = {}
        self.fused = None            # FusedExecutor on sm_100a
        self.executor = None
        self.tp = None
        self.materializer = None
        self.fsdp_grad_group = None
        self.model = None
        self.optimizer = None
        self._padding_index = None

    # ------------------------------------------------------------------ registration
    def register(self, model, mesh=None, *, sp=False):
        if self.units:
            raise RuntimeError("Runtime already registered")
        closer = getattr(mesh, "add_close_callback", None)
        if closer is not None:
            closer(self.comm.close_diagnostics)
        from shardtrain_b200.models.qwen2 import Qwen2CausalLM

        if isinstance(model, Qwen2CausalLM):
            from shardtrain_b200.runtime.qwen2_adapter import register_qwen

            return register_qwen(self, model, mesh, sp=sp)
        from shardtrain_b200.runtime.operators import register_blocks

        return register_blocks(self, model, mesh, sp=sp)

    def bind_groups(self, mesh, sp):
        """Create the TP view and the portable materialiser from a mesh (or none)."""
        self.sp = sp
        self.tp = RuntimeTPGroup(mesh.tp_group if mesh else None, self.comm,
                                 grad_group=mesh.tp_grad_group if mesh else None)
        self.materializer = Materializer(mesh.fsdp_group if mesh else None, self.comm)
        self.fsdp_grad_group = mesh.fsdp_grad_group if mesh else None
        self.defer_sp_prefetch = (self.communication_policy == "stream_ordered" and sp
                                  and self.tp.degree > 1)

    def add_parameter(self, unit, name, tp_local_value, global_shape, layout) -> ShardedParameter:
        """Plan one shard leaf.  `tp_local_value` is the CPU/GPU TP-local tensor (or a meta
        tensor when the value is filled later through `fill_shard`)."""
        spec = ParameterSpec.create(name, unit.unit_id, tp_local_value, global_shape, layout,
                                    self.materializer.degree)
        handle = ShardedParameter(spec, None, unit)
        handle.arena_offset = self.plan.add(spec)
        handle.pending_value = None if tp_local_value.device.type == "meta" else tp_local_value
        unit.handles.append(handle)
        self.registry[name] = handle
        return handle

    def allocate_arenas(self, allocator=None):
        """Create the flat parameter / gradient arenas and bind every leaf to its view."""
        total = self.plan.padded_total()
        make = allocator or (lambda n, tag: torch.zeros(n, dtype=torch.float32, device=self.device))
        self.param_arena, self.grad_arena = make(total, "param"), make(total, "grad")
        rank = self.materializer.rank
        for name, handle in self.registry.items():
            q = handle.spec.fsdp_shard_numel
            view = self.param_arena.narrow(0, handle.arena_offset, q)
            handle.local_shard = nn.Parameter(view, requires_grad=True)
            handle.grad_shard = self.grad_arena.narrow(0, handle.arena_offset, q)
            handle.grad_epoch = -1
            self.identities[name] = (id(handle.local_shard), handle.local_shard.data_ptr())
        ranges = padding_ranges(list(self.registry.values()), rank)
        self.padding_ranges = ranges
        if ranges:
            index = torch.cat([torch.arange(a, b) for a, b in ranges])
            self._padding_index = index.to(self.device)

    def sharded_parameters(self):
        return [h.local_shard for h in self.registry.values()]

    # ------------------------------------------------------------------ gradients
    def zero_grad(self):
        """Start a new accumulation window: the next commit of each leaf stores, later ones add."""
        self.grad_epoch += 1

    def first_commit(self, unit) -> bool:
        return unit.handles[0].grad_epoch != self.grad_epoch

    def mark_committed(self, handle, ticket=None):
        if handle.grad_step == self.step_id:
            raise RuntimeError(f"Repeated gradient commit {handle.spec.param_id}")
        handle.grad_step = self.step_id
        handle.grad_epoch = self.grad_epoch
        if handle.local_shard.grad is None:
            handle.local_shard.grad = handle.grad_shard
        if self.comm.streams:
            handle.grad_ready_event = ticket.ready_event if ticket is not None else torch.cuda.Event()
            if ticket is None:
                handle.grad_ready_event.record(self.comm.current_stream())
        self.comm.event("leaf_grad_committed", param_id=handle.spec.param_id,
                        unit_id=handle.spec.unit_id)

    @torch.no_grad()
    def commit_gradient(self, handle, shard_grad):
        if handle.grad_epoch != self.grad_epoch:
            handle.grad_shard.copy_(shard_grad)
        else:
            handle.grad_shard.add_(shard_grad)
        self.mark_committed(handle)

    # ------------------------------------------------------------------ optimizer binding
    def bind_optimizer(self, optimizer):
        wanted = {id(p) for p in self.sharded_parameters()}
        held = [id(p) for g in optimizer.param_groups for p in g["params"]]
        if set(held) != wanted or len(held) != len(wanted):
            raise ValueError("Optimizer must hold exactly the persistent local shards")

        def guard(opt, args, kwargs):
            if not self.active or not self.optimizer_ready or self.failed:
                raise RuntimeError("Premature optimizer: call finalize_backward first")

        def updated(opt, args, kwargs):
            self.parameter_shards_version += 1
            self.publish_parameter_shards_ready("optimizer_update")

        optimizer.register_step_pre_hook(guard)
        optimizer.register_step_post_hook(updated)
        self.optimizer = optimizer
        return optimizer

    def fused_optimizer_armed(self, unit) -> bool:
        opt = self.optimizer
        return bool(self.last_microstep and opt is not None
                    and getattr(opt, "fuse_into_reduction", False)
                    # the sm_100a reduction sums TP-replicated gradients over the mesh itself
                    and (self.fused is not None or self.tp.degree == 1
                         or all(h.spec.tp_grad_reduce == "none" for h in unit.handles)))

    def fused_optimizer_args(self):
        return self.optimizer.kernel_args()

    def note_fused_update(self, unit):
        self.optimizer.units_updated.add(unit.unit_id)

    def publish_parameter_shards_ready(self, source):
        if self.comm.streams:
            event = torch.cuda.Event()
            event.record(self.comm.current_stream())
            self.parameter_shards_ready_event = event
            if self.fused is not None:
                current = source == "optimizer_update" and getattr(
                    self.optimizer, "shadow_current", False)
                self.fused.shards_written(shadow_current=current)
        self.comm.event("parameter_shards_ready", source=source,
                        parameter_version=self.parameter_shards_version)

    def wait_parameter_shards_ready(self):
        if not self.comm.streams:
            return
        if self.parameter_shards_ready_event is None:
            raise RuntimeError("Parameter AG has no published shard readiness")
        self.comm.wait_event(self.parameter_shards_ready_event, dependency_type="DATA_DEP",
                             consumer="parameter_shards",
                             parameter_version=self.parameter_shards_version)
        if self.fused is not None:
            self.fused.before_shard_read()

    # ------------------------------------------------------------------ step boundaries
    def begin_step(self, step_id):
        if self.active or self.failed or step_id != self.step_id + 1:
            raise RuntimeError("Invalid step boundary or FAILED runtime")
        self.step_id, self.active, self.optimizer_ready = step_id, True, False
        self.comm.step_id = step_id
        if not self.comm.streams or self.parameter_shards_ready_event is None:
            self.publish_parameter_shards_ready("step_entry")
        self.backward_prefetch_tokens.clear()
        self.backward_entry_expected = self.backward_dispatch_expected = len(self.units) - 1
        for unit in self.units:
            if unit.state != "SHARDED" or (unit.lease is not None):
                raise RuntimeError(f"Live lease/state across steps U{unit.unit_id}")
            kept = self.retained_leases.pop(unit.unit_id, None)
            if kept is not None:
                # carried over from the previous micro-step of the same optimizer step
                kept.step_id = step_id
                kept.extras["carried"] = True
                unit.lease = kept
                unit.generation += 1
                kept.generation = unit.generation
            unit.forward_calls = unit.backward_calls = unit.reductions = 0
            for handle in unit.handles:
                handle.forward_uses = 0

    def prefetch(self, unit_id, phase):
        unit = self.units[unit_id]
        if unit.lease is None:
            unit.issue(phase)
        else:
            self.comm.event("prefetch_skipped_retained", unit_id=unit_id, phase=phase)

    def finalize_backward(self, *, allow_nonfinite=False):
        if not self.active or self.optimizer_ready:
            raise RuntimeError("Invalid finalize_backward boundary")
        if self.gradient_dispatch_prefetch and (
                self.backward_entry_expected != -1 or self.backward_dispatch_expected != -1):
            raise RuntimeError("Incomplete gradient-dispatch schedule")
        self.comm.finalize()
        for unit in self.units:
            if unit.state != "GRAD_READY" or unit.reductions != 1:
                raise RuntimeError(f"Missing gradient readiness U{unit.unit_id}")
        # sm_100a, a micro-step that is not the last: nothing on the compute stream reads the
        # gradient arena before the last micro-step's optimizer boundary, and the reductions of
        # the next micro-step queue behind these on the reduce-scatter stream, so the compute
        # stream does not have to stand still until the largest unit's reduction has finished
        stream_waits = not (self.fused is not None and not self.last_microstep
                            and getattr(self, "defer_gradient_check", False))
        waited = set()
        for name, handle in self.registry.items():
            if handle.grad_step != self.step_id:
                raise RuntimeError(f"Missing shard Autograd commit {name}")
            event = handle.grad_ready_event
            if stream_waits and event is not None and id(event) not in waited:
                waited.add(id(event))
                self.comm.wait_event(event, dependency_type="DATA_DEP", consumer="optimizer",
                                     param_id=name)
            grad = handle.local_shard.grad
            if grad is None or grad.shape != handle.local_shard.shape:
                raise RuntimeError(f"Missing/invalid shard .grad {name}")
        self._check_gradients(allow_nonfinite)
        if self.comm.live_buffers and not self.retained_leases:
            raise RuntimeError("Unretired buffer at optimizer boundary")
        self.optimizer_ready = True
        self.comm.event("optimizer_ready")

    def _check_gradients(self, allow_nonfinite):
        """One sweep over the gradient arena, one host read: non-finite values and padding that
        is not exactly zero (NaN/Inf in padding count as non-zero)."""
        if self.fused is not None and getattr(self, "defer_gradient_check", False):
            # every reduce-scatter kernel already checked what it wrote; the flags accumulate
            # on the device and are read together with the step metrics
            return
        if self.fused is not None:
            bad = self.fused.grad_check()
            nonfinite, padding = bool(bad[0]), bool(bad[1])
        else:
            flags = []
            if not allow_nonfinite:
                flags.append(~torch.isfinite(self.grad_arena).all())
            if self._padding_index is not None:
                flags.append(self.grad_arena[self._padding_index].count_nonzero().ne(0))
            values = torch.stack(flags).cpu().tolist() if flags else []
            nonfinite = bool(values[0]) if not allow_nonfinite and values else False
            padding = bool(values[-1]) if self._padding_index is not None and values else False
        if (nonfinite and not allow_nonfinite) or padding:
            culprit = self._locate_bad_gradient(allow_nonfinite)
            raise RuntimeError(f"Nonfinite gradient or nonzero padding {culprit}")

    def _locate_bad_gradient(self, allow_nonfinite):
        rank = self.materializer.rank
        for name, handle in self.registry.items():
            grad = handle.grad_shard
            keep = handle.spec.valid_len(rank)
            if (not allow_nonfinite and not bool(torch.isfinite(grad).all())) or bool(
                    grad[keep:].count_nonzero()):
                return name
        return "<unknown>"

    def end_step(self):
        if not self.optimizer_ready:
            raise RuntimeError("Premature optimizer/end_step")
        for name, handle in self.registry.items():
            if (id(handle.local_shard), handle.local_shard.data_ptr()) != self.identities[name]:
                raise RuntimeError(f"Shard identity/storage replaced {name}")
        for unit in self.units:
            unit.state = "SHARDED"
        self.active = False
        self.comm.event("step_end")
        self.comm.compact_completed_history()

    @contextmanager
    def compute_context(self):
        """Run the caller's step on the runtime's compute stream, joined on both sides."""
        if not self.comm.streams:
            yield
            return
        caller = self.comm.current_stream()
        compute = self.comm.streams["compute"]
        entered = torch.cuda.Event()
        entered.record(caller)
        self.comm.wait_event(entered, dependency_type="DATA_DEP", stream=compute,
                             consumer="compute_context_inputs")
        with torch.cuda.stream(compute):
            yield
        left = torch.cuda.Event()
        left.record(compute)
        self.comm.wait_event(left, dependency_type="DATA_DEP", stream=caller,
                             consumer="compute_context_outputs")

    def close(self):
        """Give back what the executor holds outside torch's allocator (peer-memory mappings).
        After a failure nothing a peer might still be reading is freed (see `PeerMemory.close`)."""
        if self.fused is not None:
            self.fused.close(failed=self.failed)

    def fail(self, reason):
        self.failed = True
        self.comm.event("runtime_failed", reason=str(reason))
        for unit in self.units:
            unit.state = "FAILED"

    # ------------------------------------------------------------------ gradient-dispatch prefetch
    @property
    def gradient_dispatch_prefetch(self):
        return (self.communication_policy == "stream_ordered" and self.sp
                and self.async_grad_rs and self.backward_prefetch)

    def _live_lease(self, unit):
        lease = unit.lease
        if lease is None or lease.step_id != self.step_id or lease.generation != unit.generation:
            raise RuntimeError(f"Missing/stale gradient-dispatch lease U{unit.unit_id}")
        return lease

    def _check_token(self, current):
        token = self.backward_prefetch_tokens.get((self.step_id, current.unit_id))
        if token is None:
            raise RuntimeError(f"Missing gradient-dispatch token U{current.unit_id}")
        target = self.units[current.unit_id - 1]
        fresh = (token["current_generation"] == current.generation
                 and token["target_unit"] == target.unit_id
                 and token["target_generation"] == target.generation
                 and token["parameter_version"] == self.parameter_shards_version)
        if not fresh:
            raise RuntimeError(f"Stale gradient-dispatch token U{current.unit_id}")
        self._live_lease(target)
        return token

    def _queue_backward_prefetch(self, current, *, owner=None):
        key = (self.step_id, current.unit_id)
        if key in self.backward_prefetch_tokens:
            raise RuntimeError(f"Duplicate gradient-dispatch token U{current.unit_id}")
        self._live_lease(current)
        target = self.units[current.unit_id - 1]
        tied = target.tied and target.unit_id == 0
        if target.forward_calls != 1 or target.reductions:
            raise RuntimeError(f"Completed/unvisited gradient-dispatch target U{target.unit_id}")
        if tied:
            ok = (target.backward_calls == 1 and target.state == "BWD_ACTIVE"
                  and len(target.handles) == 1 and target.handles[0].forward_uses == 2)
            if not ok:
                raise RuntimeError("Invalid retained tied backward target")
            self._live_lease(target)
        elif target.backward_calls or target.state not in MATERIALIZED_WAITING:
            raise RuntimeError(f"Entered/completed gradient-dispatch target U{target.unit_id}")
        elif target.lease is None:
            if target.state != "RESHARDED":
                raise RuntimeError(f"Missing retained gradient-dispatch target U{target.unit_id}")
        else:
            self._live_lease(target)
        source = "previous_gradient_dispatch" if owner is not None else "backward_gradient_dispatch_seed"
        marker = owner if owner is not None else current
        marker.annotate("BWD")
        self.comm.event("prefetch_boundary", scheduling_boundary=source,
                        gradient_owner=owner.unit_id if owner is not None else None,
                        current_unit=current.unit_id, target_unit=target.unit_id,
                        token_step=self.step_id)
        had_lease = target.lease is not None
        self.prefetch(target.unit_id, "BWD")
        token = {
            "current_generation": current.generation,
            "target_unit": target.unit_id,
            "target_generation": target.generation,
            "parameter_version": self.parameter_shards_version,
            "gradient_owner": owner.unit_id if owner is not None else None,
            "scheduling_boundary": source,
            "status": "tied_retained" if tied else "retained" if had_lease else "issued",
        }
        self.backward_prefetch_tokens[key] = token
        marker.annotate("BWD")
        self.comm.event("backward_prefetch_token", current_unit=current.unit_id, **token)

    def validate_backward_prefetch_entry(self, unit):
        if unit.tied and unit.unit_id == 0:
            if unit.state != "FWD_RETAINED":
                raise RuntimeError("Tied backward entry must retain its forward lease")
            self._live_lease(unit)
            return
        if unit.unit_id != self.backward_entry_expected:
            raise RuntimeError(f"Gradient-dispatch entry order: expected "
                               f"U{self.backward_entry_expected}, got U{unit.unit_id}")
        self._live_lease(unit)
        if unit.unit_id != len(self.units) - 1:
            self._check_token(self.units[unit.unit_id + 1])
            if unit.unit_id:
                self._check_token(unit)

    def backward_prefetch_entered(self, unit):
        if unit.tied and unit.unit_id == 0:
            self.comm.event("backward_prefetch_tied_entry", scheduling_excluded=True)
            return
        self.backward_entry_expected -= 1
        if unit.unit_id == len(self.units) - 1 and unit.unit_id:
            self._queue_backward_prefetch(unit)

    def dispatch_backward_prefetch(self, owner):
        """Called between the submission of a unit's reductions and their consumption."""
        if owner.unit_id != self.backward_dispatch_expected:
            raise RuntimeError(f"Gradient-dispatch reduction order: expected "
                               f"U{self.backward_dispatch_expected}, got U{owner.unit_id}")
        if owner.state != "GRAD_REDUCING" or owner.backward_calls != 1 or owner.reductions != 1:
            raise RuntimeError(f"Invalid gradient-dispatch owner U{owner.unit_id}")
        if owner.unit_id >= 2:
            current = self.units[owner.unit_id - 1]
            if current.backward_calls or current.reductions:
                raise RuntimeError(f"Gradient dispatch arrived after current entry U{current.unit_id}")
            if self.backward_entry_expected != current.unit_id:
                raise RuntimeError(f"Invalid gradient-dispatch frontier U{current.unit_id}")
            self._check_token(owner)
            self._queue_backward_prefetch(current, owner=owner)
        elif owner.unit_id == 0 and owner.tied:
            if self.backward_entry_expected != 0:
                raise RuntimeError("Tied reduction preceded decoder backward completion")
            self.backward_entry_expected = -1
        self.backward_dispatch_expected -= 1

    # ------------------------------------------------------------------ verification helpers
    def reported_loss(self, loss):
        self.comm.unit_id, self.comm.phase = None, "METRIC"
        value = self.tp.sum(loss.detach(), kind="loss_tp_sum") if self.sp else loss.detach().clone()
        m = self.materializer
        if m.degree > 1:
            self.comm.issue("fsdp", "loss_fsdp_sum", m.group, value, value,
                            lambda async_: dist.all_reduce(value, group=m.group, async_op=async_),
                            channel="fsdp_rs", asynchronous=False)
            value.div_(m.degree)
        return value

    def input_for_rank(self, batch):
        return self.tp.sequence_shard(batch) if self.sp else batch

    def local_loss(self, output, target):
        return (output - target).square().mean() / (self.tp.degree if self.sp else 1)

    def verification_gather(self, tensor, group, axis):
        self.comm.unit_id, self.comm.phase = None, "VERIFY"
        degree = dist.get_world_size(group) if dist.is_initialized() and group is not None else 1
        parts = [torch.empty_like(tensor) for _ in range(degree)]
        if degree == 1:
            parts[0].copy_(tensor)
        else:
            self.comm.issue(axis, "verification_ag", group, tensor, parts[0],
                            lambda async_: dist.all_gather(parts, tensor, group=group, async_op=async_),
                            channel="fsdp_ag" if axis == "fsdp" else "sp_ag", asynchronous=False,
                            extra_outputs=parts[1:])
        return parts

    def reconstruct_tp_local(self, *, gradients=False):
        """TP-local full tensors from the F shards (tests / full state dict)."""
        full = {}
        for name, handle in self.registry.items():
            shard = handle.local_shard.grad if gradients else handle.local_shard
            if shard is None:
                raise RuntimeError(f"Missing gradient {name}")
            parts = self.verification_gather(shard.detach(), self.materializer.group, "fsdp")
            flat = torch.cat([p[: handle.spec.valid_len(r)] for r, p in enumerate(parts)])
            full[name] = flat.view(handle.spec.tp_local_shape)
        return full


def _attach_qwen_api():
    """Qwen-specific methods live in qwen2_adapter; expose them as runtime methods."""
    from shardtrain_b200.runtime import qwen2_adapter as qa

    ShardedRuntime.model_forward = lambda self, model, ids, **kw: qa.model_forward(self, model, ids, **kw)
    ShardedRuntime.prepare_qwen_input = lambda self, ids, embeds: (qa.prepare_input(self, ids, embeds), None)
    ShardedRuntime.qwen_loss = lambda self, logits, labels: qa.qwen_loss(self, logits, labels)
    ShardedRuntime.qwen_reported_loss = lambda self: qa.reported_loss(self)
    ShardedRuntime.sequence_input = lambda self, t: qa.sequence_input(self, t)


_attach_qwen_api()
