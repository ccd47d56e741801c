"""Trainer of the unsharded / legacy TP-SP toy path: SGD on `output.square().mean()` with equal
micro-batches (`src/sharded_runtime/training/trainer.py:19-81`)."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor, nn


@dataclass(frozen=True)
class StepResult:
    step: int
    loss: float
    gradient_l2: float
    parameter_l2: float


def l2_norm(tensors) -> float:
    """Euclidean norm over a collection of tensors, accumulated in float64."""
    return float(torch.stack([t.detach().double().square().sum() for t in tensors]).sum().sqrt())


class Trainer:
    def __init__(self, model: nn.Module, lr: float, accumulation_steps: int = 1, *, tp_plan=None):
        if type(accumulation_steps) is not int or accumulation_steps <= 0:
            raise ValueError("accumulation_steps must be a positive integer")
        if tp_plan is not None and tp_plan.model is not model:
            raise ValueError("TP plan belongs to a different model")
        if getattr(model, "_tp_plan", None) is not tp_plan:
            raise ValueError("A converted model must be trained with its own TP/SP plan")
        self.model, self.tp_plan = model, tp_plan
        self.optimizer = torch.optim.SGD(model.parameters(), lr=lr)
        self.accumulation_steps, self.step_id = accumulation_steps, 0

    def train_step(self, batch: Tensor) -> StepResult:
        if batch.ndim != 3 or batch.shape[0] == 0 or batch.shape[0] % self.accumulation_steps:
            raise ValueError("Batch must be [B,S,H] with B divisible by accumulation_steps")
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        total = torch.zeros((), dtype=batch.dtype, device=batch.device)
        for micro in batch.chunk(self.accumulation_steps, dim=0):
            out = self.model(micro)
            loss = self.tp_plan.backward_loss(out) if self.tp_plan else out.square().mean()
            loss = loss / self.accumulation_steps
            if not torch.isfinite(loss):
                raise FloatingPointError(f"Non-finite loss at step {self.step_id}")
            loss.backward()
            total += loss.detach()
        if self.tp_plan:
            self.tp_plan.finalize_gradients()
            total = self.tp_plan.reported_loss(total)
        grads = []
        for name, p in self.model.named_parameters():
            if p.grad is None:
                raise RuntimeError(f"Missing gradient for {name} at step {self.step_id}")
            if not torch.isfinite(p.grad).all():
                raise FloatingPointError(f"Non-finite gradient for {name} at step {self.step_id}")
            grads.append(p.grad)
        grad_l2 = l2_norm(grads)   # gradients stay available until the next step
        self.optimizer.step()
        result = StepResult(self.step_id, total.item(), grad_l2, l2_norm(self.model.parameters()))
        self.step_id += 1
        return result


class ReferenceTrainer(Trainer):
    """Name kept for the unpartitioned reference path."""
