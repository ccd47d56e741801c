"""PyTorch-native comparison engine: the same Qwen2 model trained with `fully_shard` (FSDP2) only.

Nothing of this package's runtime, kernels or collectives is used here -- parameter ownership,
all-gathers and gradient reduce-scatters are PyTorch's -- so a run of this module next to
`qwen2_benchmark` separates "what the model costs on this machine" from "what the runtime adds".
It follows the reference's native baseline (`src/sharded_runtime/training/qwen2_native_baseline.py:
281-344, 392-505, 558-790`): one FSDP group per decoder layer (resharded after forward), the final
norm and the root (tied embedding / head owner) kept unsharded after forward, FP32 parameters and
FP32 gradient reduction (`MixedPrecisionPolicy(param_dtype=None, reduce_dtype=float32)`), explicit
forward / backward prefetch lists, autocast compute, AdamW(foreach=False), the same name-stable
initialisation, the same synthetic batch and the same record layout (`benchmark.rank{r}.json`,
`"engine": "native_fsdp2"`).

Scope: FSDP meshes, FSDP x TP meshes (DTensor Colwise / Rowwise plan on the projections,
`fully_shard` on the FSDP axis of a 2-D device mesh) and FSDP x TP meshes with sequence
parallelism: the residual stream, the norms, the embedding output and the logits are sharded
along the sequence (`SequenceParallel` norms, replicated DTensor embedding / head weights whose
gradients DTensor sums over the TP axis), each of the attention and MLP blocks gathers its input
ONCE for all of its column-parallel projections (compute dtype forward, FP32 for the adjoint's
reduce-scatter: `src/sharded_runtime/training/qwen2_native_baseline.py:164-278`), and the
row-parallel projections reduce-scatter their output back to the sequence shard.
"""

from __future__ import annotations

import argparse
import math
import time
from dataclasses import asdict, dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200.config import Config, ConfigError, load_config
from shardtrain_b200.distributed.context import WorkerEnvironment
from shardtrain_b200.launch.bootstrap import WorkerSession
from shardtrain_b200.models.qwen2 import causal_lm_loss_parts, rotary_inverse_frequencies
from shardtrain_b200.models.qwen2_factory import build_qwen_model
from shardtrain_b200.observability.metadata import write_json
from shardtrain_b200.runtime.qwen2_adapter import source_tensor
from shardtrain_b200.training.performance import qwen_performance_summary
from shardtrain_b200.training.qwen2_benchmark import (memory_counters, percentile,
                                                      software_versions)
from shardtrain_b200.training.qwen2_precision import resolve_qwen_compute_dtype


def materialize_same_source(model, device) -> None:
    """Replace the meta parameters by the name-stable values the sharded runtime would shard
    (one CPU tensor at a time), keeping the tied embedding / head alias."""
    tied = model.lm_head.weight is model.model.embed_tokens.weight
    for name, parameter in list(model.named_parameters()):
        value = source_tensor(model, name, parameter).to(device=device, dtype=torch.float32)
        owner = model
        *path, leaf = name.split(".")
        for part in path:
            owner = getattr(owner, part)
        owner._parameters[leaf] = torch.nn.Parameter(value)
    if tied:
        model.lm_head._parameters["weight"] = model.model.embed_tokens.weight
    # the only buffer of the model: the rotary inverse frequencies, a pure function of the config
    rotary = model.model.rotary_emb
    rotary.register_buffer("inv_freq", rotary_inverse_frequencies(
        model.config.head_dim, model.config.rope_theta, device), persistent=False)
    for name, buffer in list(model.named_buffers()):
        if buffer.device.type == "meta":
            raise RuntimeError(f"Buffer {name} cannot be materialised from a meta tensor")


def _gather_sequence_once():
    """A DTensor parallel style for a block (attention or MLP) under sequence parallelism: its
    input -- this rank's [B, S/T, H] slice -- becomes one replicated DTensor that every
    column-parallel projection inside the block consumes, so the block gathers once, not once
    per projection, and the adjoints of all projections meet in one reduce-scatter.  The gather
    moves the autocast compute dtype; the adjoint is reduced in FP32.  Only DTensor's own
    `redistribute` is used (its `forward_dtype` / `backward_dtype` arguments are what
    `PrepareModuleInput` does not expose)."""
    from torch.distributed.tensor import DTensor, Replicate, Shard
    from torch.distributed.tensor.parallel import ParallelStyle

    class GatherSequenceOnce(ParallelStyle):
        def _apply(self, module, device_mesh):
            def gather(_module, args):
                x = args[0]
                local = x if isinstance(x, DTensor) else DTensor.from_local(
                    x, device_mesh, [Shard(1)], run_check=False)
                kind = x.device.type
                forward_dtype = (torch.get_autocast_dtype(kind) if torch.is_autocast_enabled(kind)
                                 else x.dtype)
                full = local.redistribute(placements=[Replicate()], forward_dtype=forward_dtype,
                                          backward_dtype=torch.float32)
                return (full, *args[1:])

            module.register_forward_pre_hook(gather)
            return module

    return GatherSequenceOnce()


def parallelize_tensor_axis(model, tp_mesh, *, sequence_parallel: bool = False) -> None:
    """Megatron-style TP through DTensor: q/k/v/gate/up column-wise, o/down row-wise.  Without
    SP activations, norms, embedding and head stay replicated and RowwiseParallel all-reduces;
    with SP everything outside the two blocks of a layer works on this rank's sequence slice
    (see the module docstring)."""
    from torch.distributed.tensor import Replicate, Shard, distribute_tensor
    from torch.distributed.tensor.parallel import (ColwiseParallel, PrepareModuleInput,
                                                   PrepareModuleOutput, RowwiseParallel,
                                                   SequenceParallel, parallelize_module)

    degree = tp_mesh.size()
    cfg = model.config
    if (cfg.num_attention_heads % degree or cfg.num_key_value_heads % degree
            or cfg.intermediate_size % degree):
        raise ConfigError("attention heads, KV heads and the MLP width must be divisible by the "
                          "TP degree")
    row_output = Shard(1) if sequence_parallel else Replicate()
    plan = {"self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(),
            "self_attn.v_proj": ColwiseParallel(),
            "self_attn.o_proj": RowwiseParallel(output_layouts=row_output),
            "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(),
            "mlp.down_proj": RowwiseParallel(output_layouts=row_output)}
    if sequence_parallel:
        plan.update({"self_attn": _gather_sequence_once(), "mlp": _gather_sequence_once(),
                     "input_layernorm": SequenceParallel(use_local_output=True),
                     "post_attention_layernorm": SequenceParallel(use_local_output=True)})
    for layer in model.model.layers:
        parallelize_module(layer, tp_mesh, plan)
        # the module reshapes its local projection outputs: it now owns 1/T of the heads
        layer.self_attn.num_heads //= degree
        layer.self_attn.num_key_value_heads //= degree
    if not sequence_parallel:
        return
    parallelize_module(model.model.norm, tp_mesh, SequenceParallel(use_local_output=True))
    # Embedding and head: replicated weights as DTensors (one shared Parameter when tied), fed
    # with sequence-sharded DTensors, so that the weight gradient -- a partial sum over this
    # rank's positions -- is summed over the TP axis by DTensor before FSDP reduces it.
    embedding, head = model.model.embed_tokens, model.lm_head
    tied = head.weight is embedding.weight
    shared = torch.nn.Parameter(distribute_tensor(embedding.weight, tp_mesh, [Replicate()]))
    embedding.weight = shared
    head.weight = shared if tied else torch.nn.Parameter(
        distribute_tensor(head.weight, tp_mesh, [Replicate()]))
    parallelize_module(embedding, tp_mesh, PrepareModuleInput(
        input_layouts=Shard(1), desired_input_layouts=Shard(1), use_local_output=False))
    parallelize_module(embedding, tp_mesh, PrepareModuleOutput(
        output_layouts=Shard(1), desired_output_layouts=Shard(1), use_local_output=True))
    # The head is a Linear over [B, S/T, H]: DTensor would have to flatten a sharded sequence
    # dimension into the rows, which it refuses.  The rows of a linear layer are independent, so
    # the local slice goes in as the row shard of a 2-D DTensor (row order is irrelevant to the
    # weight gradient) and the local logits come back in the slice's own shape.
    from torch.distributed.tensor import DTensor

    def rows_in(_module, args):
        x = args[0]
        head._native_local_shape = x.shape[:-1]
        return (DTensor.from_local(x.reshape(-1, x.shape[-1]), tp_mesh, [Shard(0)], run_check=False),)

    def rows_out(_module, _args, out):
        return out.to_local().reshape(*head._native_local_shape, out.shape[-1])

    head.register_forward_pre_hook(rows_in)
    head.register_forward_hook(rows_out)
    rank, width = tp_mesh.get_local_rank(), None

    def slice_ids(_module, args):
        ids = args[0]
        nonlocal width
        width = ids.shape[1] // degree
        if ids.shape[1] % degree:
            raise ValueError("sequence length must be divisible by the TP degree")
        return (ids[:, rank * width:(rank + 1) * width].contiguous(), *args[1:])

    # runs before the layout hook registered above: the model hands the embedding the whole
    # [B, S] ids, the embedding sees this rank's columns
    embedding.register_forward_pre_hook(slice_ids, prepend=True)
    model._native_sequence_parallel = (rank, degree)


def shard_with_fsdp2(model, mesh, *, reshard_after_forward, forward_prefetch, backward_prefetch):
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    policy = MixedPrecisionPolicy(param_dtype=None, reduce_dtype=torch.float32)
    layers = list(model.model.layers)
    for layer in layers:
        fully_shard(layer, mesh=mesh, reshard_after_forward=reshard_after_forward, mp_policy=policy)
    fully_shard(model.model.norm, mesh=mesh, reshard_after_forward=False, mp_policy=policy)
    fully_shard(model, mesh=mesh, reshard_after_forward=False, mp_policy=policy)
    if forward_prefetch and layers:
        model.set_modules_to_forward_prefetch([layers[0]])
        for current, following in zip(layers, layers[1:] + [model.model.norm]):
            current.set_modules_to_forward_prefetch([following])
    if backward_prefetch and layers:
        model.model.norm.set_modules_to_backward_prefetch([layers[-1]])
        for index in range(1, len(layers)):
            layers[index].set_modules_to_backward_prefetch([layers[index - 1]])
    return {
        "parameter_materialization_dtype": "torch.float32",
        "gradient_reduce_dtype": "torch.float32",
        "decoder_units": len(layers),
        "decoder_reshard_after_forward": reshard_after_forward,
        "final_norm_reshard_after_forward": False,
        "root_reshard_after_forward": False,
        "explicit_forward_prefetch": forward_prefetch,
        "explicit_backward_prefetch": backward_prefetch,
        "differences": [
            "native FSDP shards dimension 0 of every parameter; this package pads the flattened "
            "TP-local tensor",
            "native FSDP2 owns its communication streams and its backward prefetch order",
        ],
    }


@dataclass
class NativeStepResult:
    step: int
    loss: float
    valid_tokens: int
    overflow: bool
    accumulation_steps: int


class NativeQwenTrainer:
    """Gradient accumulation with a global-token loss denominator, finite vote, AdamW."""

    def __init__(self, model, lr, *, dtype, optimizer, accumulation_steps, device, group,
                 loss_group=None):
        """`group`: the ranks that hold different batches (FSDP axis).  `loss_group`: the ranks
        whose loss parts add up to the global loss -- the FSDP axis, or the whole mesh when the
        sequence is sharded over the TP axis as well."""
        self.model, self.device, self.group = model, device, group
        self.loss_group = loss_group if loss_group is not None else group
        self.accumulation_steps, self.step_id = accumulation_steps, 0
        self.compute_dtype = resolve_qwen_compute_dtype(dtype, device)
        # fp16: a dynamic loss scale kept by hand (torch's GradScaler does not know that the
        # gradients are sharded DTensors whose finiteness must be voted over the mesh): start at
        # 128, halve and skip the update on overflow, double after 2000 clean steps
        # (`src/sharded_runtime/training/qwen2_native_baseline.py:392-505`).
        self.loss_scale = 128.0 if dtype == "fp16" else 1.0
        self.dynamic_scale = dtype == "fp16"
        self.growth_interval, self.clean_steps = 2000, 0
        make = {"adamw": lambda p: torch.optim.AdamW(p, lr=lr, foreach=False),
                "sgd": lambda p: torch.optim.SGD(p, lr=lr, foreach=False)}
        if optimizer not in make:
            raise ConfigError("Qwen optimizer must be sgd or adamw")
        self.optimizer = make[optimizer](model.parameters())

    def _sum(self, value, group=None):
        group = self.group if group is None else group
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(value, group=group)
        return value

    def _loss_part(self, logits, labels):
        """Summed next-token cross-entropy of this rank's logits.  Under sequence parallelism the
        logits cover this rank's positions only: the labels are shifted over the *whole*
        sequence first (the label of a slice's last position lives in the next slice)."""
        shard = getattr(self.model, "_native_sequence_parallel", None)
        if shard is None:
            return causal_lm_loss_parts(logits, labels)[0]
        rank, degree = shard
        shifted = torch.nn.functional.pad(labels[:, 1:], (0, 1), value=-100)
        width = labels.shape[1] // degree
        mine = shifted[:, rank * width:(rank + 1) * width]
        return torch.nn.functional.cross_entropy(
            logits.float().reshape(-1, logits.shape[-1]), mine.reshape(-1), ignore_index=-100,
            reduction="sum")

    def train_step(self, input_ids, labels, *, attention_mask=None, position_ids=None):
        batch = input_ids.shape[0]
        if batch % self.accumulation_steps:
            raise ValueError("batch must divide accumulation_steps")
        micro = batch // self.accumulation_steps
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        count = self._sum(labels[:, 1:].ne(-100).sum().to(torch.float64)).clamp_min(1)
        self.optimizer.zero_grad(set_to_none=True)
        total = torch.zeros((), device=self.device, dtype=torch.float64)
        enabled = self.compute_dtype != torch.float32
        for index in range(self.accumulation_steps):
            lo, hi = index * micro, (index + 1) * micro
            mask = attention_mask[lo:hi] if attention_mask is not None else None
            with torch.autocast(self.device.type, dtype=self.compute_dtype, enabled=enabled):
                out = self.model(input_ids[lo:hi], attention_mask=mask, position_ids=position_ids)
            part = self._loss_part(out.logits, labels[lo:hi])
            # FSDP averages gradients over the group: scale so the result is the global mean
            (part * (self.loss_scale * world) / count.to(part.dtype)).backward()
            total += part.detach().to(torch.float64)
        loss = self._sum(total, self.loss_group) / count
        finite = torch.isfinite(loss).to(torch.float64)
        for parameter in self.model.parameters():
            grad = parameter.grad
            if grad is not None:
                local = grad.to_local() if hasattr(grad, "to_local") else grad
                if self.loss_scale != 1.0:
                    local.mul_(1.0 / self.loss_scale)      # unscale in place before the vote
                finite = finite * torch.isfinite(local).all().to(torch.float64)
        if dist.is_initialized() and dist.get_world_size(self.loss_group) > 1:
            dist.all_reduce(finite, op=dist.ReduceOp.MIN, group=self.loss_group)
        row = torch.stack([finite, loss, count]).cpu().tolist()
        overflow = not bool(row[0])
        if not overflow:
            self.optimizer.step()
        if self.dynamic_scale:
            if overflow:                      # every rank saw the same vote: same new scale
                self.loss_scale, self.clean_steps = self.loss_scale * 0.5, 0
            else:
                self.clean_steps += 1
                if self.clean_steps == self.growth_interval:
                    self.loss_scale, self.clean_steps = self.loss_scale * 2.0, 0
        elif overflow:
            raise FloatingPointError("Nonfinite native baseline loss or gradients")
        self.step_id += 1
        return NativeStepResult(self.step_id, float(row[1]), int(row[2]), overflow,
                                self.accumulation_steps)


def run(config: Config, *, warmup: int = 0, peak_tflops_per_gpu: float | None = None) -> dict:
    """Train with FSDP2 and write `benchmark.rank{r}.json` (same timing protocol as
    `qwen2_benchmark.run`: barrier, host wall time including the device synchronise, max over
    ranks reduced outside the timer, CUDA-event span)."""
    if config.model.model_type != "qwen2":
        raise ConfigError("The native baseline requires model.model_type=qwen2")
    if config.parallel.sp_enabled and config.parallel.tp_degree < 2:
        raise ConfigError("Sequence parallelism needs a TP degree of at least 2")
    if type(warmup) is not int or warmup < 0:
        raise ConfigError("warmup must be a nonnegative integer")
    rank = WorkerEnvironment.read().rank
    if (Path(config.debug.output_dir) / f"benchmark.rank{rank}.json").exists():
        raise ConfigError(f"Output directory already contains rank {rank} experiment records; "
                          "choose a new --debug.output_dir")
    with WorkerSession(config, "runtime") as session:
        from torch.distributed.device_mesh import init_device_mesh

        ctx, tc, rc = session.context, config.training, config.runtime
        device, world = ctx.device, session.worker.world_size
        torch.manual_seed(tc.seed + rank)
        payload = {
            "engine": "native_fsdp2", "status": "initializing", "rank": rank, "world_size": world,
            "versions": software_versions(), "device": str(device), "dtype": tc.dtype,
            "optimizer": tc.optimizer, "micro_batch": tc.local_batch_size,
            "global_batch": tc.local_batch_size * tc.accumulation_steps * config.parallel.fsdp_degree,
            "sequence_length": config.model.seq_len, "accumulation_steps": tc.accumulation_steps,
            "warmup": warmup, "steady_steps_requested": tc.steps, "errors": [],
        }
        rows, failure = [], None
        try:
            model = build_qwen_model(config.model, tc.seed)
            parameters = sum(p.numel() for p in model.parameters())
            materialize_same_source(model, device)
            group = loss_group = None
            if session.worker.launched:
                degrees = (config.parallel.fsdp_degree, config.parallel.tp_degree)
                mesh = init_device_mesh(device.type, degrees, mesh_dim_names=("fsdp", "tp"))
                if degrees[1] > 1:
                    parallelize_tensor_axis(model, mesh["tp"],
                                            sequence_parallel=config.parallel.sp_enabled)
                payload["sharding"] = shard_with_fsdp2(
                    model, mesh["fsdp"], reshard_after_forward=rc.reshard_after_forward,
                    forward_prefetch=rc.forward_prefetch, backward_prefetch=rc.backward_prefetch)
                payload["sharding"]["tensor_parallel_degree"] = degrees[1]
                payload["sharding"]["sequence_parallel"] = config.parallel.sp_enabled
                group = mesh["fsdp"].get_group()      # TP ranks of a replica see the same batch
                # with SP every rank of the mesh holds a different part of the loss
                loss_group = dist.group.WORLD if config.parallel.sp_enabled else group
            trainer = NativeQwenTrainer(model, tc.lr, dtype=tc.dtype, optimizer=tc.optimizer,
                                        accumulation_steps=tc.accumulation_steps, device=device,
                                        group=group, loss_group=loss_group)
            draw = torch.Generator().manual_seed(tc.seed + ctx.coordinate.fsdp)
            ids = torch.randint(model.config.vocab_size,
                                (tc.local_batch_size * tc.accumulation_steps, config.model.seq_len),
                                generator=draw).to(device)
            labels, mask = ids.clone(), torch.ones_like(ids)
            positions = torch.arange(config.model.seq_len, device=device).unsqueeze(0)
            for _ in range(warmup):
                trainer.train_step(ids, labels, attention_mask=mask, position_ids=positions)
            if device.type == "cuda":
                torch.cuda.synchronize(device)
                torch.cuda.reset_peak_memory_stats(device)
            payload["status"] = "running"
            for index in range(tc.steps):
                if dist.is_initialized():
                    dist.barrier()
                span = None
                if device.type == "cuda":
                    span = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    span[0].record()
                t0 = time.perf_counter()
                result = trainer.train_step(ids, labels, attention_mask=mask, position_ids=positions)
                if span is not None:
                    span[1].record()
                    torch.cuda.synchronize(device)
                seconds = time.perf_counter() - t0
                slowest = torch.tensor(seconds, dtype=torch.float64, device=device)
                if dist.is_initialized() and world > 1:
                    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
                if not math.isfinite(result.loss):
                    raise FloatingPointError("Nonfinite native baseline loss")
                rows.append({**asdict(result), "measured_step": index, "seconds": seconds,
                             "max_rank_seconds": float(slowest),
                             "cuda_elapsed_ms": span[0].elapsed_time(span[1]) if span else None,
                             "tokens_per_second": result.valid_tokens / float(slowest),
                             **memory_counters(device)})
                session.logger.info("native step=%d loss=%.8f tokens=%d max_rank_seconds=%.6f",
                                    result.step, result.loss, result.valid_tokens, float(slowest))
            payload["status"] = "completed"
        except BaseException as exc:  # noqa: BLE001 - recorded, then re-raised
            failure = exc
            payload["status"] = "failed"
            payload["errors"].append(repr(exc))
        finally:
            durations = [r["max_rank_seconds"] for r in rows]
            payload.update({
                "steps": rows, "steady_steps_completed": len(rows),
                "step_seconds_p50": percentile(durations, 0.5),
                "step_seconds_p95": percentile(durations, 0.95),
                "tokens_per_second": (sum(r["valid_tokens"] for r in rows) / sum(durations)
                                      if durations else None),
                **memory_counters(device),
            })
            if rows:
                cfg = model.config
                payload["performance"] = qwen_performance_summary(
                    parameter_numel=parameters, layers=cfg.num_hidden_layers,
                    hidden_size=cfg.hidden_size, sequence_length=config.model.seq_len,
                    global_batch=payload["global_batch"], steps=rows, world_size=world,
                    peak_tflops_per_gpu=peak_tflops_per_gpu)
            write_json(session.directory / f"benchmark.rank{rank}.json", payload)
        if failure is not None:
            raise failure
        return payload


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0], allow_abbrev=False,
                                     epilog="Config overrides: --section.field value")
    parser.add_argument("--config", default="configs/qwen25_tiny.yaml")
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--peak-tflops-per-gpu", type=float, default=None)
    args, overrides = parser.parse_known_args(argv)
    try:
        run(load_config(args.config, overrides), warmup=args.warmup,
            peak_tflops_per_gpu=args.peak_tflops_per_gpu)
    except ConfigError as exc:
        parser.error(str(exc))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
