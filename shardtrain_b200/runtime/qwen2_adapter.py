"""Registration of a Qwen2 model with the sharded runtime and the runtime-driven forward.

Unit plan (reference: `src/sharded_runtime/runtime/qwen2_adapter.py:276-406`): unit 0 is the
embedding (and the LM head when tied), units 1..L the decoder layers, unit L+1 the final norm and,
for an untied model, unit L+2 the LM head.  q/k/v/gate/up are column-parallel (dim 0), o/down
row-parallel (dim 1), embedding / norms / LM head are TP-replicated; every TP-local tensor is
FSDP-sharded flat.  Each parameter is produced one at a time on the CPU (name-stable seeded
initialisation, or a slice of a safetensors checkpoint), sliced for this rank and copied into
the shard arena; the module tree keeps its Hugging Face names but its parameters become the flat
FP32 shard leaves.
"""

from __future__ import annotations

import hashlib
import json

import torch
import torch.distributed as dist
from torch.nn import functional as F

from shardtrain_b200.models.qwen2 import (
    Qwen2CausalLMOutput, apply_rotary, causal_attention, rotary_inverse_frequencies,
    rotary_tables, swiglu,
)
from shardtrain_b200.runtime.engine import TiedEmbeddingUnit, UnitState
from shardtrain_b200.runtime.qwen2_operators import (
    Branch, ColumnProjection, EmbeddingFn, NormFn, RowLinear,
)

COLUMN = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")


class ParameterPartition:
    """TP slice of a canonical tensor along `dim` (None = replicated)."""

    def __init__(self, global_shape, dim, rank, degree):
        self.global_shape, self.dim, self.rank, self.degree = tuple(global_shape), dim, rank, degree

    @property
    def local_shape(self):
        shape = list(self.global_shape)
        if self.dim is not None:
            shape[self.dim] //= self.degree
        return tuple(shape)

    def local_slice(self, tensor):
        if tuple(tensor.shape) != self.global_shape:
            raise ValueError(f"Expected logical shape {self.global_shape}, got {tuple(tensor.shape)}")
        if self.dim is None:
            return tensor
        width = self.global_shape[self.dim] // self.degree
        return tensor.narrow(self.dim, self.rank * width, width)


def seeded_parameter(model, name, shape):
    """Deterministic CPU value of one parameter, independent of creation order and of sharding:
    the generator seed is derived from the run seed and a hash of the parameter name."""
    if name.endswith(".bias"):
        return torch.zeros(shape)
    if "layernorm.weight" in name or name == "model.norm.weight":
        return torch.ones(shape)
    seed = getattr(model, "_qwen_seed", 1234)
    key = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")
    gen = torch.Generator().manual_seed((seed + key) % (2**63 - 1))
    value = torch.randn(shape, generator=gen) * model.config.initializer_range
    pad = model.config.pad_token_id
    if name == "model.embed_tokens.weight" and pad is not None:
        value[pad].zero_()
    return value


def source_tensor(model, name, parameter):
    reader = getattr(model, "_qwen_weight_source", None)
    if reader is not None:
        return reader.get_tensor(name)
    if parameter.device.type != "meta":
        return parameter.detach().cpu()
    return seeded_parameter(model, name, tuple(parameter.shape))


def initialization_digest(model) -> bytes:
    h = hashlib.sha256(json.dumps(model.config.to_dict(), sort_keys=True).encode())
    reader = getattr(model, "_qwen_weight_source", None)
    if reader is not None:
        h.update(str(reader.path).encode())
        h.update(json.dumps({k: list(v) for k, v in reader.shapes.items()}, sort_keys=True).encode())
    elif next(model.parameters()).device.type == "meta":
        h.update(str(getattr(model, "_qwen_seed", 1234)).encode())
    else:
        for name, p in model.named_parameters():
            value = p.detach().cpu().contiguous()
            h.update(name.encode())
            h.update(str(value.dtype).encode())
            h.update(value.view(torch.uint8).numpy().tobytes())
    return h.digest()


def verify_same_source(runtime, model):
    """Every rank of the TP and FSDP groups must build its shards from the same weights."""
    tp, fsdp = runtime.tp, runtime.materializer
    if tp.degree == fsdp.degree == 1:
        return
    token = torch.tensor(list(initialization_digest(model)), dtype=torch.uint8, device=runtime.device)
    differs = False
    for role, group, degree, channel in (("tp", tp.process_group, tp.degree, "sp_ag"),
                                         ("fsdp", fsdp.group, fsdp.degree, "fsdp_ag")):
        if degree > 1:
            seen = [torch.empty_like(token) for _ in range(degree)]
            runtime.comm.issue(
                role, "qwen_init_source_digest", group, token, seen[0],
                lambda async_, g=group, s=seen: dist.all_gather(s, token, group=g, async_op=async_),
                channel=channel, asynchronous=False, extra_outputs=seen[1:],
            )
            differs |= any(not torch.equal(token, other) for other in seen)
    verdict = torch.tensor(int(differs), device=runtime.device, dtype=torch.int32)
    for role, group, degree, channel in (("tp", tp.process_group, tp.degree, "sp_rs"),
                                         ("fsdp", fsdp.group, fsdp.degree, "fsdp_rs")):
        if degree > 1:
            runtime.comm.issue(
                role, "qwen_init_source_mismatch", group, verdict, verdict,
                lambda async_, g=group: dist.all_reduce(verdict, op=dist.ReduceOp.MAX, group=g,
                                                        async_op=async_),
                channel=channel, asynchronous=False,
            )
    if verdict.item():
        raise ValueError("Qwen initialization source/config differs across ranks; "
                         "use the same seed/checkpoint/weights")


_FUSED_ORDER = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                "gate_proj.weight", "up_proj.weight", "down_proj.weight",
                "q_proj.bias", "k_proj.bias", "v_proj.bias",
                "input_layernorm.weight", "post_attention_layernorm.weight")


def _fused_rank(name):
    for position, suffix in enumerate(_FUSED_ORDER):
        if name.endswith(suffix):
            return position
    return len(_FUSED_ORDER)


def _plan_parameters(model, tied):
    """(unit kind, [(hf name, owning module, attribute, tp dim)]) for every unit, in unit order."""
    core = model.model
    plan = [("embedding", [("model.embed_tokens.weight", core.embed_tokens, "weight", None)])]
    for i, layer in enumerate(core.layers):
        prefix = f"model.layers.{i}."
        entries = []
        for norm in ("input_layernorm", "post_attention_layernorm"):
            entries.append((prefix + norm + ".weight", getattr(layer, norm), "weight", None))
        for parent_name, names in (("self_attn", ("q_proj", "k_proj", "v_proj", "o_proj")),
                                   ("mlp", ("gate_proj", "up_proj", "down_proj"))):
            parent = getattr(layer, parent_name)
            for n in names:
                linear = getattr(parent, n)
                dim = 0 if n in COLUMN else 1
                entries.append((f"{prefix}{parent_name}.{n}.weight", linear, "weight", dim))
                if linear.bias is not None:
                    entries.append((f"{prefix}{parent_name}.{n}.bias", linear, "bias", 0))
        # shard arena order inside the unit = the fused layout of the sm_100a executor (matrices
        # q|k|v, o, gate|up, down, then the vectors): with FSDP degree 1 the bf16 shadow of the
        # arena then *is* the unit's materialised weight buffer and nothing has to be gathered
        entries.sort(key=lambda e: _fused_rank(e[0]))
        plan.append(("layer", entries))
    plan.append(("norm", [("model.norm.weight", core.norm, "weight", None)]))
    if not tied:
        plan.append(("head", [("lm_head.weight", model.lm_head, "weight", None)]))
    return plan


MAX_PEER_WORLD = 8      # size of the kernels' peer-pointer tables (csrc/api.h: kMaxPeers)


def fused_obstacles(runtime, cfg, mesh) -> list[str]:
    """Why the sm_100a executor cannot run this configuration (empty list: it can).

    The kernels are bf16 with 128-wide attention heads, address peers through CUDA-IPC tables of
    at most eight entries, and CUDA IPC only reaches GPUs of the same host.
    """
    reasons = []
    dtype = runtime.requested_dtype
    if dtype not in (None, "bf16"):
        reasons.append(f"compute dtype {dtype} (the sm_100a kernels are bf16 only)")
    if cfg.head_dim != 128:
        reasons.append(f"head_dim {cfg.head_dim} (the attention kernels need 128)")
    world = dist.get_world_size() if dist.is_initialized() and mesh is not None else 1
    if world > MAX_PEER_WORLD:
        reasons.append(f"{world} ranks (peer tables hold {MAX_PEER_WORLD})")
    if world > 1 and not _single_host():
        reasons.append("ranks on several hosts (CUDA IPC peer memory is per host)")
    return reasons


def _single_host() -> bool:
    import socket

    names: list = [None] * dist.get_world_size()
    dist.all_gather_object(names, socket.gethostname())
    return len(set(names)) == 1


def _choose_executor(runtime, cfg=None, mesh=None):
    """`auto`: the sm_100a executor when it can serve the configuration, else the portable one
    (with a log line saying why); `nccl`: always portable; `peer`: sm_100a or an error."""
    from shardtrain_b200 import ops

    want = runtime.communication_backend
    if runtime.device.type != "cuda" or want == "nccl":
        if want == "peer":
            raise ValueError("communication_backend: peer needs a CUDA device")
        return "portable"
    if not ops.available():
        raise RuntimeError("CUDA device requested but torch.cuda is unavailable")
    reasons = fused_obstacles(runtime, cfg, mesh) if cfg is not None else []
    if reasons:
        if want == "peer":
            raise ValueError("communication_backend: peer cannot serve this run: " + "; ".join(reasons))
        import logging

        logging.getLogger("shardtrain_b200").warning(
            "sm_100a executor not used, falling back to the portable NCCL executor: %s",
            "; ".join(reasons))
        return "portable"
    return "fused"


@torch.no_grad()
def register_qwen(runtime, model, mesh=None, *, sp=False):
    cfg = model.config
    runtime.bind_groups(mesh, sp)
    tp, fsdp = runtime.tp, runtime.materializer
    if sp and tp.degree == 1:
        raise ValueError("Qwen SP requires TP degree > 1")
    for field in ("num_attention_heads", "num_key_value_heads", "intermediate_size"):
        if getattr(cfg, field) % tp.degree:
            raise ValueError(f"Qwen {field} must be divisible by TP degree (KV replication is unsupported)")
    runtime.defer_sp_prefetch = runtime.communication_policy == "stream_ordered" and sp
    runtime.model, runtime.qwen_partitions = model, {}
    runtime.comm.phase = "INIT"
    tied = model.lm_head.weight is model.model.embed_tokens.weight
    if tied != cfg.tie_word_embeddings:
        raise ValueError("Qwen weight tying config does not match actual Parameter aliasing")
    reader = getattr(model, "_qwen_weight_source", None)
    if reader is not None:
        reader.validate({n: tuple(p.shape) for n, p in model.named_parameters(remove_duplicate=False)},
                        {"lm_head.weight": "model.embed_tokens.weight"} if tied else {})
    verify_same_source(runtime, model)

    # 1. plan every shard (no values yet) so the arenas can be sized once
    owners = {}
    for kind, entries in _plan_parameters(model, tied):
        unit_cls = TiedEmbeddingUnit if (kind == "embedding" and tied) else UnitState
        unit = unit_cls(runtime, len(runtime.units), None)
        unit.kind = kind
        runtime.units.append(unit)
        for name, module, attr, dim in entries:
            parameter = getattr(module, attr)
            part = ParameterPartition(tuple(parameter.shape), dim, tp.rank, tp.degree)
            runtime.qwen_partitions[name] = part
            shape_only = torch.empty(part.local_shape, device="meta", dtype=torch.float32)
            layout = {0: "column", 1: "row", None: "replicated"}[dim]
            handle = runtime.add_parameter(unit, name, shape_only, tuple(parameter.shape), layout)
            owners[name] = (module, attr, parameter)
    kind = _choose_executor(runtime, cfg, mesh)
    if kind == "fused":
        from shardtrain_b200.runtime.fused import FusedExecutor

        runtime.fused = FusedExecutor(runtime, model, mesh)
        runtime.fused.allocate()
        runtime.executor = runtime.fused
    else:
        runtime.allocate_arenas()
        runtime.executor = PortableQwenExecutor(runtime, model)

    # 2. one parameter at a time: CPU source -> TP slice -> this rank's FSDP shard
    for name, handle in runtime.registry.items():
        module, attr, parameter = owners[name]
        value = runtime.qwen_partitions[name].local_slice(source_tensor(model, name, parameter))
        flat = value.contiguous().reshape(-1).to(torch.float32)
        q, keep = handle.spec.fsdp_shard_numel, handle.spec.valid_len(fsdp.rank)
        if keep:
            handle.local_shard.data[:keep].copy_(flat[fsdp.rank * q : fsdp.rank * q + keep])
        if handle.spec.tp_layout == "replicated" and tp.degree > 1:
            shard = handle.local_shard.data
            runtime.comm.issue(
                "tp", "qwen_init_tp_shard", tp.process_group, shard, shard,
                lambda async_, s=shard: dist.broadcast(
                    s, src=dist.get_global_rank(tp.process_group, 0), group=tp.process_group,
                    async_op=async_),
                channel="fsdp_ag", asynchronous=False,
            )
    # 3. the module tree keeps its names; its parameters become the shard leaves
    for name, handle in runtime.registry.items():
        module, attr, _ = owners[name]
        module._parameters[attr] = handle.local_shard
    if tied:
        model.lm_head._parameters["weight"] = runtime.registry["model.embed_tokens.weight"].local_shard
    for i, layer in enumerate(model.model.layers):
        unit = runtime.units[1 + i]
        unit.block = layer
        prefix = f"model.layers.{i}."
        unit.forward_prefetch_handle = runtime.registry[prefix + "self_attn.v_proj.weight"]
        unit.backward_prefetch_handle = runtime.registry[prefix + "mlp.down_proj.weight"]
    runtime.units[0].block = model.model.embed_tokens
    runtime.units[0].forward_prefetch_handle = runtime.registry["model.embed_tokens.weight"]
    norm_unit = runtime.units[1 + len(model.model.layers)]
    norm_unit.block = model.model.norm
    norm_unit.forward_prefetch_handle = norm_unit.backward_prefetch_handle = runtime.registry["model.norm.weight"]
    runtime.inv_freq = rotary_inverse_frequencies(cfg.head_dim, cfg.rope_theta, runtime.device)
    runtime.local_heads = cfg.num_attention_heads // tp.degree
    runtime.local_kv_heads = cfg.num_key_value_heads // tp.degree
    runtime.tied = tied
    if not hasattr(runtime, "compute_dtype"):
        runtime.compute_dtype = torch.float32
    model._sharded_runtime = runtime
    model.__dict__.pop("_qwen_weight_source", None)
    if runtime.fused is not None:
        runtime.fused.finish_registration()
    return runtime


class PortableQwenExecutor:
    """Qwen2 unit math with torch ops and the portable consumers (CPU/gloo, NCCL baseline)."""

    name = "portable"

    def __init__(self, runtime, model):
        self.runtime, self.cfg = runtime, model.config

    def embedding(self, unit, ids):
        handle = unit.handle("model.embed_tokens.weight")
        weight = unit.forward_weight(handle.spec.param_id)
        return EmbeddingFn.apply(ids, weight, handle, self.cfg.pad_token_id)

    def norm(self, unit, name, x):
        handle = unit.handle(name)
        return NormFn.apply(x, unit.forward_weight(name), handle, self.cfg.rms_norm_eps)

    def _column_group(self, unit, prefix, names, x, role):
        runtime = self.runtime
        branches, weights = [], []
        for n in names:
            w = unit.handle(f"{prefix}{n}.weight")
            b = runtime.registry.get(f"{prefix}{n}.bias")
            branches.append(Branch(w, b))
            weights.append(unit.forward_weight(w.spec.param_id))
            if b is not None:
                weights.append(unit.forward_weight(b.spec.param_id))
        boundary = branches[-1].weight
        with runtime.tp.tagged(role):
            return ColumnProjection.apply(x, runtime, tuple(branches), boundary, *weights)

    def _row(self, unit, name, x, *, replicated=False, tied_second_use=False):
        handle = unit.handle(name)
        weight = unit.forward_weight(name, tied_second_use=tied_second_use)
        return RowLinear.apply(x, weight, self.runtime, handle, replicated)

    def layer(self, unit, index, x, tables, attention_mask):
        runtime = self.runtime
        p = f"model.layers.{index}."
        d = self.cfg.head_dim
        h = self.norm(unit, p + "input_layernorm.weight", x)
        q, k, v = self._column_group(unit, p + "self_attn.", ("q_proj", "k_proj", "v_proj"), h, "qkv")
        batch, seq, _ = q.shape

        def heads(t, n):
            return t.reshape(batch, seq, n, d).transpose(1, 2)

        q, k, v = heads(q, runtime.local_heads), heads(k, runtime.local_kv_heads), heads(v, runtime.local_kv_heads)
        cos, sin = tables
        if cos.shape[-2] != seq:
            raise ValueError("QKV sequence length differs from global RoPE positions")
        q, k = apply_rotary(q, k, cos, sin)
        cd = runtime.compute_dtype
        mixed = causal_attention(q.to(cd), k.to(cd), v.to(cd), attention_mask)
        mixed = mixed.transpose(1, 2).reshape(batch, seq, -1)
        x = x + self._row(unit, p + "self_attn.o_proj.weight", mixed)
        h = self.norm(unit, p + "post_attention_layernorm.weight", x)
        gate, up = self._column_group(unit, p + "mlp.", ("gate_proj", "up_proj"), h, "gate_up")
        return x + self._row(unit, p + "mlp.down_proj.weight", swiglu(gate, up))

    def final_norm(self, unit, x):
        return self.norm(unit, "model.norm.weight", x)

    def head_loss(self, unit, hidden, labels, *, tied):
        name = "model.embed_tokens.weight" if tied else "lm_head.weight"
        logits = self._row(unit, name, hidden, replicated=True, tied_second_use=tied)
        return logits, None


def prepare_input(runtime, ids, embeds):
    if embeds is not None:
        raise ValueError("ShardTrain Qwen training requires token IDs; inputs_embeds is reference-only")
    if ids is None or ids.ndim != 2:
        raise ValueError("Qwen token IDs must have shape [batch, global sequence]")
    if runtime.sp and ids.shape[1] % runtime.tp.degree:
        raise ValueError("Qwen global sequence must be divisible by TP degree for SP")
    runtime.qwen_global_seq = ids.shape[1]
    return sequence_input(runtime, ids)


def sequence_input(runtime, tensor):
    """This rank's sequence slice of a [B, S, ...] tensor under SP (the tensor itself otherwise)."""
    if not runtime.sp:
        return tensor
    if tensor.ndim < 2 or tensor.shape[1] % runtime.tp.degree:
        raise ValueError("Qwen sequence tensors must divide TP degree on dimension 1")
    width = tensor.shape[1] // runtime.tp.degree
    return tensor.narrow(1, runtime.tp.rank * width, width).clone()


def sum_metric(runtime, value, kind):
    """SUM of a scalar over the SP group (when SP) and the FSDP group."""
    fused = getattr(runtime, "fused", None)
    if fused is not None and fused.reduce_peer.degree > 1:
        # sm_100a executor: one kernel over peer memory (with SP the TP ranks hold different
        # sequence slices, so the sum runs over F x T; without SP over the FSDP group only)
        total = fused.metric_peer.all_reduce_small(value.detach().to(torch.float64).reshape(1))
        if runtime.comm.diagnostics_enabled:
            runtime.comm.event("metric_allreduce", kind=kind, backend="peer_kernel")
        return total[0].to(value.dtype)
    result = value.detach().clone()
    hops = []
    if runtime.sp:
        hops.append(("tp", runtime.tp.process_group, runtime.tp.degree, "sp_rs"))
    m = runtime.materializer
    hops.append(("fsdp", m.group, m.degree, "fsdp_rs"))
    for role, group, degree, channel in hops:
        if degree > 1:
            runtime.comm.issue(
                role, f"{kind}_{role}", group, result, result,
                lambda async_, g=group: dist.all_reduce(result, group=g, async_op=async_),
                channel=channel, asynchronous=False,
            )
    return result


def shifted_labels(runtime, labels):
    """Next-token targets; the shift happens before SP slicing so the token across a shard
    boundary is the right one."""
    if labels.ndim != 2 or labels.shape[1] != runtime.qwen_global_seq:
        raise ValueError("Qwen labels must describe the full global sequence")
    return sequence_input(runtime, F.pad(labels[:, 1:], (0, 1), value=-100))


def qwen_loss(runtime, logits, labels):
    target = shifted_labels(runtime, labels)
    if target.shape != logits.shape[:2]:
        raise ValueError("Qwen logits/label shard shape mismatch")
    total = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), target.reshape(-1),
                            ignore_index=-100, reduction="sum")
    return finish_loss(runtime, total, target.ne(-100).sum())


def finish_loss(runtime, total, local_count):
    override = getattr(runtime, "qwen_denominator_override", None)
    denom = sum_metric(runtime, local_count, "lm_valid_count") if override is None else override
    runtime.qwen_denominator = denom.clamp_min(1)
    runtime.qwen_numerator = total.detach()
    # the reduce-scatter averages over F once; scale so the result is the global token mean
    return total * runtime.materializer.degree / runtime.qwen_denominator


def reported_loss(runtime):
    return sum_metric(runtime, runtime.qwen_numerator, "lm_loss_sum") / runtime.qwen_denominator


def model_forward(runtime, model, input_ids, *, attention_mask=None, position_ids=None,
                  labels=None, inputs_embeds=None, default_positions=False):
    """Walk the units in order with materialised weights (called by `Qwen2CausalLM.forward`)."""
    ex = runtime.executor
    ids = prepare_input(runtime, input_ids, inputs_embeds)
    units, layers = runtime.units, model.model.layers
    tied = runtime.tied
    first = units[0]
    first.pre_forward()
    hidden = ex.embedding(first, ids)
    if tied:
        first.embedding_complete()
    else:
        hidden = first.post_forward(hidden)
    tables = ex.rotary(position_ids, default_positions) if hasattr(ex, "rotary") else rotary_tables(
        position_ids.to(hidden.device), runtime.inv_freq, hidden.dtype)
    for index in range(len(layers)):
        unit = units[1 + index]
        unit.pre_forward()
        with torch.profiler.record_function(f"shardtrain/qwen/layer{index}"):
            hidden = ex.layer(unit, index, hidden, tables, attention_mask)
        hidden = unit.post_forward(hidden)
    unit = units[1 + len(layers)]
    unit.pre_forward()
    hidden = unit.post_forward(ex.final_norm(unit, hidden))
    head_unit = first if tied else units[-1]
    if not tied:
        head_unit.pre_forward()
    logits, loss = ex.head_loss(head_unit, hidden, labels, tied=tied)
    out = logits if logits is not None else loss
    out = first.head_complete(out) if tied else head_unit.post_forward(out)
    if logits is not None:
        logits, loss = out, (qwen_loss(runtime, out, labels) if labels is not None else None)
    else:
        loss = out
    return Qwen2CausalLMOutput(logits=logits, loss=loss, last_hidden_state=hidden)
