"""sm_100a executor: the Qwen2 units computed with this package's CUDA kernels only.

Per unit, the `PeerMaterializer` lands the gathered parameters already cast to bf16 in one flat
buffer whose order is chosen for the kernels: `q|k|v` weights adjacent (one QKV GEMM), `gate|up`
adjacent (one gate/up GEMM), small vectors (biases, norm weights) in an FP32 side buffer.  The
backward writes every parameter gradient in FP32 straight into one slot of a peer-visible ring
(`GradRing`) laid out the same way, so the reduce-scatter kernel can pull this rank's slice of
every peer's slot without any packing pass, average it, accumulate it into the gradient arena
and, on the last micro-step, apply AdamW in the same pass.

One decoder layer is one autograd node (`FusedLayerFn`): forward and backward are explicit
sequences of kernel launches (RMSNorm, tcgen05 GEMMs with fused bias / residual epilogues, RoPE,
tcgen05 attention, SwiGLU), saving only compact activations.  The residual stream stays FP32,
GEMM operands are bf16, accumulation is FP32 -- the same precision plan as the reference under
bf16 autocast (`src/sharded_runtime/runtime/qwen2_operators.py:39-204`).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch.autograd.function import once_differentiable

from shardtrain_b200 import ops as ops_module
from shardtrain_b200.distributed.peer import CHANNEL_SLOTS, PeerMemory
from shardtrain_b200.runtime.layout import segment_table
from shardtrain_b200.runtime.materializer import PeerMaterializer

SP_FLAG_SLOT = CHANNEL_SLOTS["sp_ag"]    # barrier flag slot of the in-stream SP barriers

_LAYER_ORDER = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                "gate_proj.weight", "up_proj.weight", "down_proj.weight",
                "q_proj.bias", "k_proj.bias", "v_proj.bias",
                "input_layernorm.weight", "post_attention_layernorm.weight")


def _up(value, multiple):
    return -(-value // multiple) * multiple


@dataclass
class UnitPlan:
    """Where each parameter of a unit lives in the materialised buffers and in the gradient slot."""

    names: list[str] = field(default_factory=list)
    shapes: dict[str, tuple] = field(default_factory=dict)
    param_offsets: dict[str, int] = field(default_factory=dict)   # into the bf16 or fp32 buffer
    fp32_names: set[str] = field(default_factory=set)
    grad_offsets: dict[str, int] = field(default_factory=dict)    # into the fp32 gradient slot
    bf16_numel: int = 0
    fp32_numel: int = 0
    grad_numel: int = 0
    shard_numel: int = 0
    gather_table: torch.Tensor | None = None
    reduce_table: torch.Tensor | None = None
    # decoder layers: the gather table split for the "pull the weights inside the GEMM" forward
    # -- rows of q|k|v and of gate|up (consumed by the fused all-gather GEMMs) and the rest (o,
    # down and the vectors, still landed by the gather kernel)
    ag_segs_qkv: torch.Tensor | None = None
    ag_segs_gu: torch.Tensor | None = None
    gather_table_rest: torch.Tensor | None = None
    # persistent materialisation state (allocated once at registration)
    full_bf16: torch.Tensor | None = None
    full_fp32: torch.Tensor | None = None
    weights: dict = field(default_factory=dict)      # name -> view of the buffers above
    tokens: tuple = ()                                # one-element FP32 autograd edge tokens
    last_reader: object = None                        # event after the buffers' last consumer
    fwd: dict = field(default_factory=dict)           # fused operand views (built on first use)
    gslots: dict = field(default_factory=dict)        # id(slot) -> fused gradient views

    def views(self, full_bf16, full_fp32):
        out = {}
        for name in self.names:
            shape = self.shapes[name]
            n = math.prod(shape)
            src = full_fp32 if name in self.fp32_names else full_bf16
            out[name] = src.narrow(0, self.param_offsets[name], n).view(shape)
        return out

    def span(self, buffer, first, last, cols):
        """Contiguous 2-D view covering parameters first..last (adjacent in the layout)."""
        start = self.param_offsets[first]
        stop = self.param_offsets[last] + math.prod(self.shapes[last])
        return buffer.narrow(0, start, stop - start).view(-1, cols)

    def grad_view(self, slot, name):
        return slot.narrow(0, self.grad_offsets[name], math.prod(self.shapes[name])).view(self.shapes[name])

    def grad_span(self, slot, first, last, cols):
        start = self.grad_offsets[first]
        stop = self.grad_offsets[last] + math.prod(self.shapes[last])
        return slot.narrow(0, start, stop - start).view(-1, cols)


def build_plan(unit) -> UnitPlan:
    plan = UnitPlan()
    by_name = {h.spec.param_id: h for h in unit.handles}

    def rank_of(name):
        for position, suffix in enumerate(_LAYER_ORDER):
            if name.endswith(suffix):
                return position
        return len(_LAYER_ORDER)

    ordered = sorted(by_name, key=lambda n: (rank_of(n), unit.handles.index(by_name[n])))
    plan.names = ordered
    bf16_cursor = fp32_cursor = grad_cursor = 0
    for name in ordered:
        spec = by_name[name].spec
        plan.shapes[name] = spec.tp_local_shape
        if len(spec.tp_local_shape) == 1:
            plan.fp32_names.add(name)
            plan.param_offsets[name] = fp32_cursor
            fp32_cursor = _up(fp32_cursor + spec.numel, 4)
        else:
            plan.param_offsets[name] = bf16_cursor
            bf16_cursor = _up(bf16_cursor + spec.numel, 8)
        plan.grad_offsets[name] = grad_cursor
        grad_cursor = _up(grad_cursor + spec.numel, 4)
        plan.shard_numel += spec.fsdp_shard_numel
    plan.bf16_numel, plan.fp32_numel, plan.grad_numel = bf16_cursor, fp32_cursor, grad_cursor
    handles = [by_name[n] for n in ordered]
    plan.gather_table = segment_table(handles, plan.param_offsets, plan.fp32_names)
    plan.reduce_table = segment_table(handles, plan.grad_offsets, set(), mark_replicated=True)
    # Only gate|up (88 % of a layer's pulled bytes, a GEMM wide enough to occupy every SM) is
    # left to the pulling GEMM.  q|k|v stays with the gather kernel: its weight has too few rows
    # to spread over the machine (measured 49 us pulled inside the GEMM against 27 us for gather
    # kernel + GEMM at 512 x 2048 x 1536), so `ag_segs_qkv` stays unset.
    gu = [i for i, n in enumerate(ordered) if n.endswith(_LAYER_ORDER[4:6])]
    if len(gu) == 2:
        rest = [i for i in range(len(ordered)) if i not in gu]
        plan.ag_segs_gu = plan.gather_table[gu].contiguous()
        plan.gather_table_rest = plan.gather_table[rest].contiguous()
    return plan


class GradSlot:
    def __init__(self, local, peer_ptrs, multicast_ptr=0):
        self.local, self.peer_ptrs, self.multicast_ptr = local, peer_ptrs, multicast_ptr
        self.holder = None
        self.last_rs = -10


class GradRing:
    """Peer-visible FP32 slots the backward writes full gradients into.

    A slot may be overwritten once the reduce-scatter that consumed it has finished on this GPU
    *and* every peer has finished pulling from it.  The second condition holds once this rank's
    next reduce-scatter barrier has passed (a peer enters barrier n+1 only after its pull n), so
    a slot last used by reduction n is handed out again after waiting for the event of
    reduction n+1.
    """

    def __init__(self, peer: PeerMemory, ops, numel: int, count: int = 4, multicast: bool = False):
        """`multicast`: ask for slots that are also reachable through an NVLS multicast address
        (falls back to plain peer memory when the fabric refuses)."""
        self.slots = []
        for _ in range(count):
            buf = peer.alloc_multicast(numel * 4) if multicast else peer.alloc(numel * 4)
            self.slots.append(GradSlot(buf.tensor(ops, numel) if peer.degree > 1
                                       else buf.owner.view(torch.float32)[:numel], buf.ptrs,
                                       buf.multicast_ptr))
        self.events: list = []      # events[n]: completion of reduction n on the rs stream

    def acquire(self, unit_id, stream):
        free = [s for s in self.slots if s.holder is None]
        if not free:
            raise RuntimeError("No free gradient slot (a unit's reduction was never issued)")
        slot = min(free, key=lambda s: s.last_rs)
        guard = slot.last_rs + 1
        if slot.last_rs >= 0:
            event = self.events[min(guard, len(self.events) - 1)]
            stream.wait_event(event)
        slot.holder = unit_id
        return slot

    def issued(self, slot, event):
        slot.last_rs = len(self.events)
        slot.holder = None
        self.events.append(event)
        if len(self.events) > 4096:   # keep indices stable but drop old events
            cut = len(self.events) - 64
            self.events = [None] * cut + self.events[cut:]


class FusedExecutor:
    name = "fused"

    def __init__(self, runtime, model, mesh):
        self.runtime, self.cfg, self.mesh = runtime, model.config, mesh
        if self.cfg.head_dim != 128:
            raise ValueError("The sm_100a attention kernel supports head_dim 128 only")
        self.ops = ops_module.load()
        self.status = self.ops.status_tensor()
        wait = runtime.device_wait_seconds
        self.peer = PeerMemory(mesh.fsdp_group if mesh else None, runtime.device, self.ops,
                               wait_seconds=wait)
        # With a TP axis: activations travel inside the TP group, gradient slots are visible to
        # the whole mesh (TP-replicated parameters are summed over all of it).
        self.tp_degree, self.tp_rank = runtime.tp.degree, runtime.tp.rank
        if self.tp_degree > 1:
            import torch.distributed as dist

            self.tp_peer = PeerMemory(mesh.tp_group, runtime.device, self.ops, wait_seconds=wait)
            self.reduce_peer = PeerMemory(dist.group.WORLD, runtime.device, self.ops,
                                          wait_seconds=wait)
            if self.reduce_peer.degree != self.peer.degree * self.tp_degree:
                raise ValueError("The mesh must cover the whole world (F * T ranks)")
        else:
            self.tp_peer, self.reduce_peer = None, self.peer
        self._sp_buffers = {}
        self._tp_buffers = {}
        self.exp_avg = self.exp_avg_sq = None
        self._shards_dirty = True
        self.shards_clean_event = None
        self._flags = torch.zeros(2, dtype=torch.int32, device=runtime.device)
        self.check_flags = self._flags   # written by every reduce-scatter kernel
        self._rope_cache = {}
        self._mask_cache = {}
        self._scratch = {}
        self.token_grad = torch.zeros(1, dtype=torch.float32, device=runtime.device)
        self.rows_hint = None     # rows of the layer GEMMs' activation, known after the first input
        # Replay of a layer's launch sequence as a CUDA graph (FSDP-only meshes: the TP / SP
        # sequences carry barrier epochs that change at every call).  `_forward_open` holds the
        # layers whose forward has run and whose backward has not: their activations live in
        # buffers the replay cache owns, so a second forward before the backward must not replay.
        self.replay = bool(runtime.cuda_graphs) and self.tp_degree == 1
        self._forward_open = set()

    # ------------------------------------------------------------------ fused all-gather -> GEMM
    # `auto` pulls only where one pass over the weights serves every row tile (four 128-row
    # accumulators in TMEM) AND nothing else would hide the gather.  Measured on B200, gate|up of
    # Qwen2.5-1.5B with 8 owners: kernel against kernel the fused GEMM wins at 512 rows (62 us
    # against 65 us gather kernel + gated GEMM on 8 GPUs) and loses at 1024 rows (111 / 84 us);
    # inside the training step with forward prefetch the gather kernel runs on its own stream
    # under the previous layer's compute, while the fused GEMM puts the pull on the compute
    # stream: F8T1 on 8 GPUs 61.1 ms per step with the pull, 60.1 ms without.
    PULL_MAX_ROWS = 512

    def pulls_in_gemm(self, unit, phase) -> bool:
        """Should this materialisation leave q|k|v and gate|up to the consuming GEMMs?  Only in
        the forward of a decoder layer, with FSDP peers to pull from; `auto` also wants the
        activation to fit the accumulators the kernel keeps in TMEM in one pass (<= 512 rows)
        and forward prefetch to be off (with prefetch the gather is already hidden)."""
        mode = self.runtime.fused_allgather
        plan = self.runtime.materializer.plans[unit.unit_id]
        if mode == "off" or phase != "FWD" or self.peer.degree == 1 or plan.ag_segs_gu is None:
            return False
        if mode == "on":
            return True
        return (not self.runtime.forward_prefetch and self.rows_hint is not None
                and self.rows_hint <= self.PULL_MAX_ROWS)

    def ag_arguments(self, unit, plan):
        """The five trailing arguments of the layer-forward ops: empty unless this lease left
        q|k|v and gate|up in the owners' arenas for the GEMMs to pull."""
        if not unit.lease.extras.get("pull_in_gemm"):
            return [], False, None, None, None
        fp32 = self.runtime.wire_dtype == "fp32"
        arenas = self.param_peer_ptrs if fp32 else self.shadow_peer_ptrs
        return list(arenas), fp32, plan.ag_segs_qkv, plan.ag_segs_gu, plan.full_bf16

    # ------------------------------------------------------------------ allocation
    def allocate(self):
        rt = self.runtime
        portable = rt.materializer
        mat = PeerMaterializer(portable.group, rt.comm, self.peer)
        total = rt.plan.padded_total()
        self._param_buffer = self.peer.alloc(total * 4)

        def make(n, tag):
            if tag == "param":
                if self.peer.degree > 1:
                    return self._param_buffer.tensor(self.ops, n)
                return self._param_buffer.owner.view(torch.float32)[:n]
            return torch.zeros(n, dtype=torch.float32, device=rt.device)

        rt.materializer = mat
        rt.allocate_arenas(allocator=make)
        self.param, self.grad = rt.param_arena, rt.grad_arena
        self.param_peer_ptrs = list(self._param_buffer.ptrs)
        # compute-dtype shadow of the shard arena (same element offsets): written by the fused
        # AdamW kernel next to the FP32 master, read by the peers' gather kernels
        self._shadow_buffer = self.peer.alloc(total * 2)
        self.shadow = (self._shadow_buffer.tensor(self.ops, total, torch.bfloat16)
                       if self.peer.degree > 1
                       else self._shadow_buffer.owner.view(torch.bfloat16)[:total])
        self.shadow_peer_ptrs = list(self._shadow_buffer.ptrs)
        self._shadow_stale = True
        largest = 0
        token_pool = torch.zeros(64 * max(1, len(rt.units)), dtype=torch.float32, device=rt.device)
        for unit in rt.units:
            plan = mat.plans[unit.unit_id] = build_plan(unit)
            largest = max(largest, plan.grad_numel)
            if self._alias_shadow(unit, plan):
                # FSDP degree 1: a "gathered" matrix is the shard itself, and the shadow arena
                # already holds it in bf16 at the offsets the kernels want -- the unit's weight
                # buffer is a window of the shadow, only the FP32 vectors are still copied
                lo = rt.plan.unit_ranges[unit.unit_id][0]
                plan.full_bf16 = self.shadow.narrow(0, lo, max(plan.bf16_numel, 8))
                keep = plan.gather_table[:, 4].bitwise_and(1).ne(0)
                plan.gather_table = plan.gather_table[keep].contiguous()
            else:
                plan.full_bf16 = torch.empty(max(plan.bf16_numel, 8), dtype=torch.bfloat16,
                                             device=rt.device)
            plan.full_fp32 = torch.empty(max(plan.fp32_numel, 4), dtype=torch.float32, device=rt.device)
            plan.weights = plan.views(plan.full_bf16, plan.full_fp32)
            base = 64 * unit.unit_id
            if len(unit.handles) > 64:
                raise ValueError("A unit may hold at most 64 parameters")
            plan.tokens = tuple(token_pool[base + i: base + i + 1] for i in range(len(unit.handles)))
        # NVLS reduce-scatter: only where the multicast group is exactly the FSDP group (no TP
        # axis) -- with TP the slots are shared by the whole mesh and a multicast sum would add
        # the other TP coordinates' gradients of TP-split parameters
        want_nvls = (rt.nvls != "off" and self.tp_degree == 1 and self.peer.degree > 1)
        self.ring = GradRing(self.reduce_peer, self.ops, _up(largest, 4), count=4,
                             multicast=want_nvls)
        self.nvls_active = all(slot.multicast_ptr for slot in self.ring.slots) and want_nvls
        mat.bind(self.ops, self)
        ranges = rt.padding_ranges or [(0, 0)]
        self._pad_ranges = torch.tensor(ranges, dtype=torch.int64, device=rt.device).reshape(-1)

    def _alias_shadow(self, unit, plan) -> bool:
        """True when the unit's bf16 matrices sit in the shard arena exactly as in its fused
        weight buffer (single FSDP member, matrices first and in fused order)."""
        if self.peer.degree != 1:
            return False
        lo = self.runtime.plan.unit_ranges[unit.unit_id][0]
        matrices = [h for h in unit.handles if h.spec.param_id not in plan.fp32_names]
        return bool(matrices) and all(
            h.arena_offset - lo == plan.param_offsets[h.spec.param_id] for h in matrices)

    def close(self, *, failed=False):
        """Unmap and free the peer-visible buffers (arenas, gradient ring, activation slots).
        Tensors that alias them (`param`, `grad` views, shard leaves) must not be used
        afterwards.  With `failed` nothing is freed: a peer may still be reading."""
        if self.replay and not failed:
            # the replay cache keeps this executor's activations and graphs alive: give them back
            # (the cache is per process; another executor's entries are simply rebuilt)
            torch.cuda.synchronize(self.runtime.device)
            self.ops.replay_clear()
        seen = set()
        for peer in (self.tp_peer, self.reduce_peer, self.peer):
            if peer is not None and id(peer) not in seen:
                seen.add(id(peer))
                peer.close(failed=failed)

    def finish_registration(self):
        rt = self.runtime
        self.hq, self.hkv = rt.local_heads, rt.local_kv_heads
        torch.cuda.synchronize(rt.device)

    def state_arena(self, tag):
        t = torch.zeros_like(self.param)
        setattr(self, tag, t)
        return t

    # ------------------------------------------------------------------ runtime hooks
    def shards_written(self, shadow_current=False):
        """The FP32 shards changed.  `shadow_current`: every write went through a kernel that
        also wrote the bf16 shadow (the fused reduce-scatter + AdamW); otherwise the shadow is
        rebuilt from the masters before the next gather."""
        self._shards_dirty = True
        if not shadow_current:
            self._shadow_stale = True

    def before_shard_read(self):
        """Runs on the gather stream before the first gather after the shards changed."""
        if self._shards_dirty:
            if self._shadow_stale:
                self.ops.cast_bf16(self.param, self.shadow)
                self._shadow_stale = False
            self.peer.barrier("fsdp_ag")
            self._shards_dirty = False
            # readers of the peers' shards on OTHER streams (the embedding lookup) wait for this
            self.shards_clean_event = torch.cuda.Event()
            self.shards_clean_event.record(self.runtime.comm.current_stream())

    def acquire_grad_slot(self, unit):
        if getattr(unit, "grad_slot", None) is None:
            unit.grad_slot = self.ring.acquire(unit.unit_id, self.runtime.comm.current_stream())
        return unit.grad_slot

    def grad_slot(self, unit):
        slot = getattr(unit, "grad_slot", None)
        if slot is None:
            raise RuntimeError(f"U{unit.unit_id} reduced without a gradient slot")
        return slot

    def grad_slot_issued(self, unit, slot, ticket):
        self.ring.issued(slot, ticket.ready_event)
        unit.grad_slot = None

    def layer_operands(self, plan, index):
        """Fused operand views of a decoder layer's persistent buffers (built once)."""
        if not plan.fwd:
            p = f"model.layers.{index}."
            wb, wf = plan.full_bf16, plan.full_fp32
            H = self.cfg.hidden_size
            W = (self.hq + 2 * self.hkv) * 128
            inter = plan.shapes[p + "mlp.gate_proj.weight"][0]
            plan.fwd = dict(
                w_qkv=plan.span(wb, p + "self_attn.q_proj.weight", p + "self_attn.v_proj.weight", H),
                b_qkv=wf.narrow(0, plan.param_offsets[p + "self_attn.q_proj.bias"], W),
                w_o=plan.span(wb, p + "self_attn.o_proj.weight", p + "self_attn.o_proj.weight", self.hq * 128),
                w_gu=plan.span(wb, p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight", H),
                w_down=plan.span(wb, p + "mlp.down_proj.weight", p + "mlp.down_proj.weight", inter),
                ln1=wf.narrow(0, plan.param_offsets[p + "input_layernorm.weight"], H),
                ln2=wf.narrow(0, plan.param_offsets[p + "post_attention_layernorm.weight"], H),
                inter=inter, width=W,
            )
        return plan.fwd

    def layer_gradients(self, plan, slot, index):
        """Fused gradient views of a decoder layer inside one ring slot (built once per slot)."""
        views = plan.gslots.get(id(slot))
        if views is None:
            p = f"model.layers.{index}."
            g = slot.local
            H = self.cfg.hidden_size
            W = (self.hq + 2 * self.hkv) * 128
            views = plan.gslots[id(slot)] = dict(
                down=plan.grad_view(g, p + "mlp.down_proj.weight"),
                gate_up=plan.grad_span(g, p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight", H),
                ln2=plan.grad_view(g, p + "post_attention_layernorm.weight"),
                o=plan.grad_view(g, p + "self_attn.o_proj.weight"),
                bias=g.narrow(0, plan.grad_offsets[p + "self_attn.q_proj.bias"], W),
                qkv=plan.grad_span(g, p + "self_attn.q_proj.weight", p + "self_attn.v_proj.weight", H),
                ln1=plan.grad_view(g, p + "input_layernorm.weight"),
            )
        return views

    def sp_buffers(self, batch, seq, layers):
        """Peer-visible activation buffers of the sequence-parallel layers for one input shape:
        per layer the bf16 h1 / h2 slices (read in place by the peers' gathers and by the
        backward's re-gathers), two bf16 gradient slices, and T fp32 receive slots the row GEMMs'
        epilogues scatter into.  Allocation is collective over the TP group (same order on every
        member), happens once per shape and is never freed before shutdown."""
        key = (batch, seq)
        buf = self._sp_buffers.get(key)
        if buf is None:
            T, H, tp = self.tp_degree, self.cfg.hidden_size, self.tp_peer
            rows = batch * (seq // T)
            act_bytes, slot_bytes = rows * H * 2, rows * H * 4
            acts = tp.alloc(layers * 2 * act_bytes)
            grads = tp.alloc(2 * act_bytes)
            recv = tp.alloc(T * slot_bytes)
            bf = torch.bfloat16

            def act(layer, which):
                off = (layer * 2 + which) * act_bytes
                return (acts.tensor(self.ops, rows * H, bf, off).view(rows, H),
                        [p + off for p in acts.ptrs])

            buf = dict(
                h=[(act(i, 0), act(i, 1)) for i in range(layers)],
                dob=(grads.tensor(self.ops, rows * H, bf, 0).view(rows, H), list(grads.ptrs)),
                dmb=(grads.tensor(self.ops, rows * H, bf, act_bytes).view(rows, H),
                     [p + act_bytes for p in grads.ptrs]),
                recv=recv.tensor(self.ops, T * rows * H, torch.float32).view(T, rows, H),
                # where this rank's partial rows for owner p go: p's slot number tp_rank
                push=[p + self.tp_rank * slot_bytes for p in recv.ptrs],
                flags=list(tp.flags.ptrs),
            )
            self._sp_buffers[key] = buf
        return buf

    def tp_buffers(self, batch, seq):
        """Receive sets of the all-reduce used by tensor parallelism without SP: two alternating
        sets of T fp32 [batch*seq, H] slots per rank, peer visible; `push_x[p]` is where this
        rank's partial rows go in member p's set."""
        key = (batch, seq)
        buf = self._tp_buffers.get(key)
        if buf is None:
            T, H, tp = self.tp_degree, self.cfg.hidden_size, self.tp_peer
            rows = batch * seq
            slot_bytes = rows * H * 4
            sets = [tp.alloc(T * slot_bytes) for _ in range(2)]
            buf = dict(
                recv=[b.tensor(self.ops, T * rows * H, torch.float32).view(T, rows, H) for b in sets],
                push=[[p + self.tp_rank * slot_bytes for p in b.ptrs] for b in sets],
                flags=list(tp.flags.ptrs),
            )
            self._tp_buffers[key] = buf
        return buf

    @property
    def metric_peer(self):
        """Group over which per-step sums run: with SP the TP ranks hold different sequence
        slices (whole mesh); without SP they hold identical values (FSDP group only)."""
        return self.reduce_peer if (self.runtime.sp or self.tp_degree == 1) else self.peer

    def launch_grad_check(self):
        self.ops.grad_check(self.grad, self._pad_ranges, self._flags)

    def grad_check(self):
        self.launch_grad_check()
        flags = self._flags.cpu().tolist()
        self._flags.zero_()
        return flags

    def scratch(self, key, shape, dtype):
        t = self._scratch.get(key)
        if t is None or t.shape != torch.Size(shape) or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.runtime.device)
            self._scratch[key] = t
        return t

    def key_mask_bits(self, attention_mask):
        """Packed form of a [batch, sequence] key mask (one bit per key, int32 [B, pitch]) for
        the attention kernels.  The bits live in ONE buffer per mask shape, refilled when another
        mask tensor (or another version of it) arrives: every layer of a micro-step presents the
        same mask, so the packing runs once per micro-step at most, and the buffer's address --
        part of a layer's replay key -- stays the same from step to step even when the caller
        builds a fresh mask tensor every step."""
        if attention_mask.ndim != 2:
            raise ValueError("The sm_100a attention kernel takes a [batch, sequence] key mask")
        batch, seq = attention_mask.shape
        source = (attention_mask.data_ptr(), attention_mask._version)
        bits = self.scratch(("key_mask_bits", batch, seq), (batch, 4 * ((seq + 127) // 128)), torch.int32)
        held = self._mask_cache.get((batch, seq))
        if held is None or held[0] != source:
            as_bytes = attention_mask.to(self.runtime.device).ne(0).to(torch.uint8).contiguous()
            self.ops.pack_key_mask(as_bytes, bits)
            # the entry keeps the caller's tensor alive: its address cannot be reused meanwhile
            self._mask_cache[(batch, seq)] = (source, attention_mask)
        return bits

    def rotary(self, position_ids, default_positions):
        """cos/sin tables (FP32, [rows, D/2]) for the RoPE kernel and an optional int32 row index
        per (batch, token).  Default positions 0..S-1 and a caller-supplied [1, S] row share one
        table of S rows indexed by `token % S`; per-sample positions [B, S] get a table of B*S rows
        indexed by the token's row.  Tables of caller-supplied positions are cached on the
        tensor's identity and version, so a batch that repeats them pays once; they are rebuilt
        in place when fresh positions arrive."""
        seq = position_ids.shape[-1]
        inv_freq = self.runtime.inv_freq.float()
        if default_positions:
            key = ("default", seq)
            if key not in self._rope_cache:
                pos = torch.arange(seq, device=self.runtime.device, dtype=torch.float32)
                angle = pos[:, None] * inv_freq[None, :]
                self._rope_cache[key] = (angle.cos().contiguous(), angle.sin().contiguous(), None)
        else:
            # One set of tables per shape of `position_ids`, at fixed addresses (they are part of
            # a layer's replay key), recomputed when another tensor or version arrives.
            shape = tuple(position_ids.shape)
            key = ("given", shape)
            source = (position_ids.data_ptr(), position_ids._version)
            held = self._rope_cache.get(key)
            if held is None or held[3] != source:
                pos = position_ids.to(self.runtime.device, torch.float32).reshape(-1)
                angle = pos[:, None] * inv_freq[None, :]
                cos = self.scratch(("rope_cos", shape), tuple(angle.shape), torch.float32)
                sin = self.scratch(("rope_sin", shape), tuple(angle.shape), torch.float32)
                torch.cos(angle, out=cos)
                torch.sin(angle, out=sin)
                rows = None
                if position_ids.shape[0] != 1:
                    rows = self.scratch(("rope_rows", shape), (pos.numel(),), torch.int32)
                    torch.arange(pos.numel(), out=rows)
                # the entry keeps `position_ids` alive, so its address cannot be handed to another
                # tensor while the entry is current
                self._rope_cache[key] = (cos, sin, rows, source, position_ids)
        cos, sin, rows = self._rope_cache[key][:3]
        return cos, sin, rows, seq

    # ------------------------------------------------------------------ unit math
    def embedding(self, unit, ids):
        handle = unit.handle("model.embed_tokens.weight")
        weight = unit.forward_weight(handle.spec.param_id)
        return FusedEmbeddingFn.apply(weight, ids, self, unit)

    def layer(self, unit, index, x, tables, attention_mask):
        plan = self.runtime.materializer.plans[unit.unit_id]
        weights = [unit.forward_weight(n) for n in plan.names]
        mask = self.key_mask_bits(attention_mask) if attention_mask is not None else None
        return FusedLayerFn.apply(x, self, unit, index, tables, mask, *weights)

    def final_norm(self, unit, x):
        weight = unit.forward_weight("model.norm.weight")
        return FusedNormFn.apply(x, weight, self, unit)

    def head_loss(self, unit, hidden, labels, *, tied):
        name = "model.embed_tokens.weight" if tied else "lm_head.weight"
        if tied:
            # the embedding lookup did not wait for the gathered table (it reads the shards);
            # the head is its first reader
            self.runtime.materializer.await_deferred(unit)
        weight = unit.forward_weight(name, tied_second_use=tied)
        if labels is None:
            raise ValueError("The sm_100a executor fuses the LM head with the loss; pass labels")
        loss = FusedHeadLossFn.apply(hidden, weight, self, unit, name, labels)
        return None, loss


# ---------------------------------------------------------------------------- autograd nodes
class FusedEmbeddingFn(torch.autograd.Function):
    """Embedding rows read straight from the (possibly remote) FP32 shards: no table gather is
    needed for the lookup.  Backward scatter-adds into the unit's gradient slot."""

    @staticmethod
    def forward(ctx, weight, ids, ex, unit):
        rt = ex.runtime
        handle = unit.handles[0]
        ctx.ex, ctx.unit = ex, unit
        ctx.save_for_backward(ids)
        hidden = ex.cfg.hidden_size
        flat = ids.reshape(-1).contiguous()
        ex.rows_hint = flat.numel() * (ex.tp_degree if rt.sp else 1)
        ex._forward_open.clear()          # a new micro-step's forward begins here
        if ex.replay:
            # same address at every micro-step, so the first layer's replay key repeats
            # (a fresh view each time: autograd attaches this call's node to the object it gets)
            out = ex.scratch("embedding_out", (*ids.shape, hidden), torch.float32).view(*ids.shape, hidden)
        else:
            out = torch.empty((*ids.shape, hidden), dtype=torch.float32, device=rt.device)
        base = handle.arena_offset * 4
        ptrs = [p + base for p in ex.param_peer_ptrs]
        ex.ops.embedding_gather_sharded(ptrs, handle.spec.fsdp_shard_numel, flat, out)
        unit.prefetch_after_input(handle, "FWD")
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        ex, unit = ctx.ex, ctx.unit
        unit.annotate("BWD")
        (ids,) = ctx.saved_tensors
        handle = unit.handles[0]
        name = handle.spec.param_id
        plan = ex.runtime.materializer.plans[unit.unit_id]
        fresh = getattr(unit, "grad_slot", None) is None
        slot = ex.acquire_grad_slot(unit)
        dw = plan.grad_view(slot.local, name)
        if fresh:
            dw.zero_()  # untied: nothing wrote the slot yet; tied: the head's dW is already there
        pad = ex.cfg.pad_token_id
        ex.ops.embedding_scatter_add(grad.reshape(-1, grad.shape[-1]).contiguous(),
                                     ids.reshape(-1).contiguous(), dw, -1 if pad is None else pad)
        # a tied weight receives its gradient view from the head node; returning it twice would
        # make autograd add the two (identical) views
        return (None if unit.tied else ex.token_grad), None, None, None


class FusedNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, ex, unit):
        ctx.ex, ctx.unit = ex, unit
        unit.annotate("FWD")
        hidden = x.shape[-1]
        weight = unit.lease.weights[unit.handles[0].spec.param_id]   # `weight` is only the edge token
        x2 = x.reshape(-1, hidden).contiguous()
        y = torch.empty(x2.shape, dtype=torch.bfloat16, device=x.device)
        inv = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        ex.ops.rmsnorm_fwd(x2, weight, y, inv, ex.cfg.rms_norm_eps)
        ctx.save_for_backward(x2, inv)
        ctx.shape = x.shape
        unit.prefetch_after_input(unit.handles[0], "FWD")
        return y.view(x.shape)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        ex, unit = ctx.ex, ctx.unit
        unit.annotate("BWD")
        x2, inv = ctx.saved_tensors
        name = unit.handles[0].spec.param_id
        weight = unit.weight(name)
        plan = ex.runtime.materializer.plans[unit.unit_id]
        slot = ex.acquire_grad_slot(unit)
        side = ex.__dict__.pop("_head_dx", None)   # FP32 gradient handed over by the head node
        dy = side if side is not None else grad.reshape(x2.shape).float().contiguous()
        dx = (ex.scratch("final_norm_dx", x2.shape, x2.dtype) if ex.replay
              else torch.empty_like(x2))      # a stable address for the last layer's replay key
        partial = ex.scratch("norm_partial", (592, x2.shape[1]), torch.float32)
        ex.ops.rmsnorm_bwd(dy, x2, weight, inv, None, dx, partial)
        dw = plan.grad_view(slot.local, name)
        ex.ops.colsum_f32(partial, dw, False)
        return dx.view(ctx.shape), ex.token_grad, None, None


class FusedHeadLossFn(torch.autograd.Function):
    """LM head GEMM + vocabulary cross-entropy.  Logits live in one reused bf16 buffer, are
    turned into their own gradient in place, and feed the dW / dX GEMMs."""

    @staticmethod
    def forward(ctx, hidden, weight, ex, unit, name, labels):
        from shardtrain_b200.runtime.qwen2_adapter import finish_loss, shifted_labels

        rt, ops = ex.runtime, ex.ops
        unit.annotate("FWD")
        ctx.ex, ctx.unit, ctx.name = ex, unit, name
        h = hidden.shape[-1]
        weight = unit.lease.weights[name]   # the `weight` argument is only the autograd edge token
        hidden2 = hidden.reshape(-1, h)
        rows, vocab = hidden2.shape[0], weight.shape[0]
        target = shifted_labels(rt, labels).reshape(-1).contiguous()
        logits = ex.scratch("logits", (rows, vocab), torch.bfloat16)
        ops.gemm(hidden2, weight, logits, False, False, None, None, False, 1.0, 0)
        lse = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        per_row = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        ops.ce_fwd(logits, target, lse, per_row)
        total = torch.empty(1, dtype=torch.float32, device=hidden.device)
        ops.sum_f32(per_row, total, False)
        loss = finish_loss(rt, total[0], target.ne(-100).sum())
        ctx.factor = rt.materializer.degree / rt.qwen_denominator
        ctx.save_for_backward(hidden2, target, lse)
        ctx.hidden_shape = hidden.shape
        return loss

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        ex, unit, name = ctx.ex, ctx.unit, ctx.name
        ops = ex.ops
        unit.annotate("BWD")
        hidden2, target, lse = ctx.saved_tensors
        weight = unit.weight(name)
        rows, vocab = hidden2.shape[0], weight.shape[0]
        logits = ex.scratch("logits", (rows, vocab), torch.bfloat16)
        scale = (grad.float() * ctx.factor).reshape(1).contiguous()
        ops.ce_bwd(logits, target, lse, scale)
        plan = ex.runtime.materializer.plans[unit.unit_id]
        slot = ex.acquire_grad_slot(unit)
        dw = plan.grad_view(slot.local, name)
        ops.gemm(logits, hidden2, dw, True, True, None, None, False, 1.0, 0)
        dx = torch.empty(hidden2.shape, dtype=torch.float32, device=hidden2.device)
        ops.gemm(logits, weight, dx, False, True, None, None, False, 1.0, 0)
        ex._head_dx = dx
        placeholder = torch.empty(ctx.hidden_shape, dtype=torch.bfloat16, device=hidden2.device)
        return placeholder, ex.token_grad, None, None, None, None


class FusedLayerFn(torch.autograd.Function):
    """One decoder layer: 4 GEMMs forward, 8 backward, everything else in fused kernels."""

    @staticmethod
    def forward(ctx, x, ex, unit, index, tables, mask, *weights):
        ops, cfg = ex.ops, ex.cfg
        plan = ex.runtime.materializer.plans[unit.unit_id]
        unit.annotate("FWD")
        if unit.lease is None or unit.state != "FWD_ACTIVE":
            raise RuntimeError("Layer forward without a current materialization")
        w = ex.layer_operands(plan, index)
        B, S, H = x.shape
        M, D, hq, hkv = B * S, 128, ex.hq, ex.hkv
        W, inter = w["width"], w["inter"]
        cos, sin, positions, _ = tables
        dev = x.device
        x2 = x.reshape(M, H).contiguous()
        w_qkv, b_qkv, w_o, w_gu, w_down, ln1, ln2 = (
            w["w_qkv"], w["b_qkv"], w["w_o"], w["w_gu"], w["w_down"], w["ln1"], w["ln2"])
        unit.prefetch_after_input(unit.forward_prefetch_handle, "FWD")
        ctx.ex, ctx.unit, ctx.index, ctx.tables, ctx.mask = ex, unit, index, tables, mask
        ag = ex.ag_arguments(unit, plan)
        # after this forward the unit's full buffer is complete either way (the pulling GEMMs
        # mirror what they pull), so later readers of the lease take the plain path
        unit.lease.extras["pull_in_gemm"] = False
        if ex.tp_degree > 1 and not ex.runtime.sp:
            # tensor parallel, replicated activations: partial sums are all-reduced by push
            tp = ex.tp_peer
            buf = ex.tp_buffers(B, S)
            epoch = tp.epochs["sp_ag"]
            h1, inv1, qkv, attn, lse, x_mid, h2, inv2, gu, out, hm = ops.layer_forward_tp(
                x2, w_qkv, b_qkv, w_o, w_gu, w_down, ln1, ln2, cos, sin, positions, mask,
                ex.status, B, S, hq, hkv, cfg.rms_norm_eps, buf["push"][0], buf["push"][1],
                buf["recv"][0], buf["recv"][1], buf["flags"], ex.tp_rank, epoch, SP_FLAG_SLOT,
                tp.wait_us, *ag)
            tp.epochs["sp_ag"] = epoch + 2
            ctx.dims = (B, S, H, inter)
            ctx.save_for_backward(x2, inv1, h1, qkv, attn, lse, x_mid, inv2, h2, gu, hm)
            return out.view(B, S, H)
        if ex.tp_degree > 1:
            # sequence parallel: x is this rank's [B, S/T, H] slice of the residual stream
            T, tp = ex.tp_degree, ex.tp_peer
            S_full = S * T
            buf = ex.sp_buffers(B, S_full, cfg.num_hidden_layers)
            (h1, h1_ptrs), (h2, h2_ptrs) = buf["h"][index]
            epoch = tp.epochs["sp_ag"]
            inv1, qkv, attn, lse, x_mid, inv2, gu, out, hm = ops.layer_forward_sp(
                x2, w_qkv, b_qkv, w_o, w_gu, w_down, ln1, ln2, cos, sin, positions, mask,
                ex.status, B, S_full, hq, hkv, cfg.rms_norm_eps, h1, h2, h1_ptrs, h2_ptrs,
                buf["push"], buf["recv"], buf["flags"], ex.tp_rank, epoch, SP_FLAG_SLOT,
                tp.wait_us, ex.runtime.fused_seq_gather, *ag)
            tp.epochs["sp_ag"] = epoch + 4
            ctx.dims = (B, S_full, H, inter)
            ctx.save_for_backward(x2, inv1, qkv, attn, lse, x_mid, inv2, gu, hm)
            return out.view(B, S, H)
        # the 10 launches of the forward run from C++ (csrc/layer_executor.cpp)
        replay = ex.replay and index not in ex._forward_open
        if ex.replay and torch.is_grad_enabled():
            ex._forward_open.add(index)
        ctx.replay = replay
        h1, inv1, qkv, attn, lse, x_mid, h2, inv2, gu, out, hm = ops.layer_forward(
            x2, w_qkv, b_qkv, w_o, w_gu, w_down, ln1, ln2, cos, sin, positions, mask, ex.status,
            B, S, hq, hkv, cfg.rms_norm_eps, *ag, replay)

        ctx.dims = (B, S, H, inter)
        ctx.save_for_backward(x2, inv1, h1, qkv, attn, lse, x_mid, inv2, h2, gu, hm)
        return out.view(B, S, H)

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        ex, unit, index = ctx.ex, ctx.unit, ctx.index
        ops = ex.ops
        plan = ex.runtime.materializer.plans[unit.unit_id]
        unit.annotate("BWD")
        unit.weight(plan.names[0])  # state / generation check of the backward materialisation
        if ex.tp_degree > 1 and ex.runtime.sp:
            return FusedLayerFn._backward_sp(ctx, dout, plan)
        x2, inv1, h1, qkv, attn, lse, x_mid, inv2, h2, gu, hm = ctx.saved_tensors
        B, S, H, inter = ctx.dims
        M, D, hq, hkv = B * S, 128, ex.hq, ex.hkv
        cos, sin, positions, _ = ctx.tables
        bf, f32 = torch.bfloat16, torch.float32
        w = ex.layer_operands(plan, index)
        W = w["width"]
        w_qkv, w_o, w_gu, w_down, ln1, ln2 = w["w_qkv"], w["w_o"], w["w_gu"], w["w_down"], w["ln1"], w["ln2"]
        slot = ex.acquire_grad_slot(unit)
        gv = ex.layer_gradients(plan, slot, index)
        unit.prefetch_after_input(unit.backward_prefetch_handle, "BWD")

        d_out = dout.reshape(M, H).contiguous()
        if ex.tp_degree > 1:
            tp = ex.tp_peer
            buf = ex.tp_buffers(B, S)
            epoch = tp.epochs["sp_ag"]
            dx = ops.layer_backward_tp(
                d_out, x2, inv1, h1, qkv, attn, lse, x_mid, inv2, h2, gu, hm, w_qkv, w_o, w_gu,
                w_down, ln1, ln2, gv["down"], gv["gate_up"], gv["ln2"], gv["o"], gv["bias"],
                gv["qkv"], gv["ln1"], cos, sin, positions, ctx.mask, ex.status, B, S, hq, hkv,
                buf["push"][0], buf["push"][1], buf["recv"][0], buf["recv"][1], buf["flags"],
                ex.tp_rank, epoch, SP_FLAG_SLOT, tp.wait_us)
            tp.epochs["sp_ag"] = epoch + 2
            return (dx.view(B, S, H), None, None, None, None, None,
                    *([ex.token_grad] * len(plan.names)))
        # the 26 launches of the backward run from C++ (csrc/layer_executor.cpp)
        dx = ops.layer_backward(
            d_out, x2, inv1, h1, qkv, attn, lse, x_mid, inv2, h2, gu, hm, w_qkv, w_o, w_gu, w_down, ln1,
            ln2, gv["down"], gv["gate_up"], gv["ln2"], gv["o"], gv["bias"], gv["qkv"], gv["ln1"], cos,
            sin, positions, ctx.mask, ex.status, B, S, hq, hkv, ctx.replay)
        ex._forward_open.discard(index)
        return (dx.view(B, S, H), None, None, None, None, None, *([ex.token_grad] * len(plan.names)))

    @staticmethod
    def _backward_sp(ctx, dout, plan):
        ex, unit, index = ctx.ex, ctx.unit, ctx.index
        ops, tp = ex.ops, ex.tp_peer
        x2, inv1, qkv, attn, lse, x_mid, inv2, gu, hm = ctx.saved_tensors
        B, S_full, H, inter = ctx.dims
        cos, sin, positions, _ = ctx.tables
        w = ex.layer_operands(plan, index)
        slot = ex.acquire_grad_slot(unit)
        gv = ex.layer_gradients(plan, slot, index)
        unit.prefetch_after_input(unit.backward_prefetch_handle, "BWD")
        buf = ex.sp_buffers(B, S_full, ex.cfg.num_hidden_layers)
        (_, h1_ptrs), (_, h2_ptrs) = buf["h"][index]
        (dob, dob_ptrs), (dmb, dmb_ptrs) = buf["dob"], buf["dmb"]
        rows = x2.shape[0]
        d_out = dout.reshape(rows, H).contiguous()
        epoch = tp.epochs["sp_ag"]
        dx = ops.layer_backward_sp(
            d_out, x2, inv1, qkv, attn, lse, x_mid, inv2, gu, hm, w["w_qkv"], w["w_o"], w["w_gu"],
            w["w_down"], w["ln1"], w["ln2"], gv["down"], gv["gate_up"], gv["ln2"], gv["o"],
            gv["bias"], gv["qkv"], gv["ln1"], cos, sin, positions, ctx.mask, ex.status, B, S_full,
            ex.hq, ex.hkv, dob, dmb, h1_ptrs, h2_ptrs, dob_ptrs, dmb_ptrs, buf["push"], buf["recv"],
            buf["flags"], ex.tp_rank, epoch, SP_FLAG_SLOT, tp.wait_us, ex.runtime.fused_seq_gather)
        tp.epochs["sp_ag"] = epoch + 4
        return (dx.view(B, S_full // ex.tp_degree, H), None, None, None, None, None,
                *([ex.token_grad] * len(plan.names)))
