"""Causal-LM training step over the sharded runtime: micro-batch accumulation with a global
token denominator, compute-dtype selection, fp16 loss scaling with a rank-wide finite vote, one
batched host read of (finite, loss, valid tokens) per optimizer step.

Semantics follow `src/sharded_runtime/training/qwen2_trainer.py:36-193`: each micro-batch is a
full runtime step (its own gathers and reductions), the loss of every micro-batch is divided by
the number of valid labels of the *whole* optimizer step across all ranks, non-finite gradients
raise in fp32/bf16 and skip the update with a scale back-off in fp16, and any exception moves the
runtime to `FAILED`.  The optimizer is a flat-arena one (`training/optim.py`).
"""

from __future__ import annotations

import time
from contextlib import contextmanager
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch.nn import functional as F

from shardtrain_b200.runtime.qwen2_adapter import sequence_input, sum_metric
from shardtrain_b200.training.optim import ArenaAdamW, ArenaSGD
from shardtrain_b200.training.qwen2_precision import resolve_qwen_compute_dtype


@contextmanager
def training_range(name, device):
    label = "shardtrain/qwen/" + name
    with torch.profiler.record_function(label):
        cuda = torch.device(device).type == "cuda"
        if cuda:
            torch.cuda.nvtx.range_push(label)
        try:
            yield
        finally:
            if cuda:
                torch.cuda.nvtx.range_pop()


@dataclass
class QwenStepResult:
    step: int
    loss: float
    valid_tokens: int
    overflow: bool
    loss_scale: float
    accumulation_steps: int


class QwenTrainer:
    def __init__(self, model, runtime, lr=0.001, *, dtype="fp32", optimizer="sgd",
                 accumulation_steps=1, fuse_optimizer=None):
        self.compute_dtype = resolve_qwen_compute_dtype(dtype, runtime.device)
        if accumulation_steps < 1:
            raise ValueError("accumulation_steps must be positive")
        if runtime.fused is not None and dtype != "bf16":
            # the sm_100a executor computes in bf16 whatever the trainer asks for: refuse rather
            # than train silently in another precision than the one configured
            raise ValueError(
                f"training dtype {dtype} on the sm_100a executor, whose kernels are bf16 only: "
                "construct ShardedRuntime(compute_dtype=...) with the training dtype (the portable "
                "executor is then selected) or set runtime.communication_backend: nccl")
        runtime.compute_dtype = self.compute_dtype
        self.model, self.runtime, self.dtype = model, runtime, dtype
        self.accumulation_steps, self.step_id = accumulation_steps, 0
        self.blocked_seconds = 0.0    # host time spent waiting in the per-step metric read
        if optimizer == "sgd":
            self.optimizer = ArenaSGD(runtime, lr=lr)
        elif optimizer == "adamw":
            self.optimizer = ArenaAdamW(runtime, lr=lr)
        else:
            raise ValueError("Qwen optimizer must be sgd or adamw")
        runtime.bind_optimizer(self.optimizer)
        if fuse_optimizer is None:
            fuse_optimizer = runtime.fused is not None and optimizer == "adamw" and dtype != "fp16"
        self.optimizer.fuse_into_reduction = bool(fuse_optimizer and runtime.fused is not None)
        runtime.defer_gradient_check = runtime.fused is not None
        self.scaler = torch.amp.GradScaler("cuda", enabled=dtype == "fp16", init_scale=128.0)

    # ------------------------------------------------------------------ metrics
    def _finite_vote(self, reported):
        """1 if every rank's gradients (and the loss) are finite, as an int32 device tensor."""
        runtime = self.runtime
        if runtime.fused is not None:
            # written by the gradient-check kernel of every micro-step
            finite = runtime.fused._flags[0].eq(0).to(torch.int32)
        else:
            finite = torch.isfinite(runtime.grad_arena).all().to(torch.int32)
        finite.mul_(torch.isfinite(reported).to(torch.int32))
        runtime.comm.unit_id, runtime.comm.phase = None, "AMP"
        if runtime.fused is not None and runtime.fused.reduce_peer.degree > 1:
            voted = runtime.fused.reduce_peer.all_reduce_small(
                finite.to(torch.float64).reshape(1), min_mask=1)
            return voted[0].to(torch.int32)
        m = runtime.materializer
        for role, group, degree, channel in (("tp", runtime.tp.process_group, runtime.tp.degree, "sp_rs"),
                                             ("fsdp", m.group, m.degree, "fsdp_rs")):
            if degree > 1:
                runtime.comm.issue(
                    role, "amp_finite_" + role, group, finite, finite,
                    lambda async_, g=group: dist.all_reduce(finite, op=dist.ReduceOp.MIN, group=g,
                                                            async_op=async_),
                    channel=channel, asynchronous=False,
                )
        return finite

    def _read_metrics(self, reported, global_count):
        finite = self._finite_vote(reported)
        fused = self.runtime.fused
        padding = fused._flags[1] if fused is not None else torch.zeros((), device=finite.device)
        # the kernels' status word (bounded waits that expired, rejected arguments) rides along in
        # the same device-to-host read, so a silent peer fails this very step on the host
        status = fused.status[0] if fused is not None else torch.zeros((), device=finite.device)
        packed = torch.stack([finite.to(torch.float64), reported.detach().to(torch.float64),
                              global_count.to(torch.float64), padding.to(torch.float64),
                              status.to(torch.float64)])
        began = time.perf_counter()
        row = packed.cpu().tolist()          # the step's one device-to-host read
        self.blocked_seconds += time.perf_counter() - began
        if fused is not None:
            fused._flags.zero_()
            if row[4]:
                from shardtrain_b200 import ops as ops_module

                ops_module.check_status("in train_step")
        if row[3]:
            raise RuntimeError("Nonzero gradient padding in a shard")
        return bool(row[0]), float(row[1]), int(row[2])

    # ------------------------------------------------------------------ step
    def train_step(self, input_ids, labels=None, *, attention_mask=None, position_ids=None):
        runtime = self.runtime
        labels = input_ids if labels is None else labels
        batch = input_ids.shape[0]
        if labels.shape != input_ids.shape or batch % self.accumulation_steps:
            raise ValueError("Labels must match input IDs and batch must divide accumulation_steps")
        micro = batch // self.accumulation_steps
        total = torch.zeros((), device=runtime.device)
        with runtime.compute_context():
            try:
                runtime.zero_grad()
                runtime.comm.unit_id, runtime.comm.phase = None, "METRIC"
                runtime.qwen_global_seq = input_ids.shape[1]
                target = sequence_input(runtime, F.pad(labels[:, 1:], (0, 1), value=-100))
                global_count = sum_metric(runtime, target.ne(-100).sum(), "lm_accum_valid_count")
                runtime.qwen_denominator_override = global_count.clamp_min(1)
                for index in range(self.accumulation_steps):
                    lo, hi = index * micro, (index + 1) * micro

                    def part(value):
                        return value[lo:hi] if value is not None and value.shape[0] == batch else value

                    runtime.last_microstep = index + 1 == self.accumulation_steps
                    runtime.begin_step(runtime.step_id + 1)
                    with training_range("model_forward", runtime.device):
                        out = self.model(input_ids[lo:hi], attention_mask=part(attention_mask),
                                         position_ids=part(position_ids), labels=labels[lo:hi])
                    total.add_(runtime.qwen_numerator)
                    with training_range("backward", runtime.device):
                        self.scaler.scale(out.loss).backward()
                        # A non-finite shard gradient is not raised here, on the one rank that
                        # happens to hold it: that rank would leave the step before the metric
                        # collectives and its peers would only learn of it from a broken
                        # connection or a timeout.  The finite vote below makes every rank raise
                        # (bf16 / fp32) or skip the update (fp16) in the same step.
                        runtime.finalize_backward(allow_nonfinite=True)
                    if not runtime.last_microstep:
                        runtime.end_step()
                    del out
                runtime.qwen_numerator = total
                runtime.comm.unit_id, runtime.comm.phase = None, "METRIC"
                reported = runtime.qwen_reported_loss()
                if self.scaler.is_enabled():
                    self.scaler.unscale_(self.optimizer)
                finite, loss_value, valid = self._read_metrics(reported, global_count)
                scale = None
                with training_range("optimizer", runtime.device):
                    if finite:
                        self.scaler.step(self.optimizer)
                        self.scaler.update()
                    elif self.scaler.is_enabled():
                        # every rank skips the same update and adopts the same scale
                        scale = self.scaler.get_scale() * self.scaler.get_backoff_factor()
                        self.scaler.update(new_scale=scale)
                        state = self.scaler.state_dict()
                        scale, state["_growth_tracker"] = state["scale"], 0
                        self.scaler.load_state_dict(state)
                    else:
                        raise RuntimeError("Nonfinite Qwen loss/gradients")
                runtime.end_step()
                if scale is None:
                    scale = self.scaler.get_scale()
                result = QwenStepResult(self.step_id, loss_value, valid, not finite, scale,
                                        self.accumulation_steps)
                self.step_id += 1
                return result
            except BaseException as exc:
                runtime.fail(exc)
                raise
            finally:
                runtime.__dict__.pop("qwen_denominator_override", None)
                runtime.last_microstep = True
