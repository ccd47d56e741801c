"""SGD trainer of the unsharded toy path and of the legacy TP/SP plan: loss
`output.square().mean()`, equal micro-batches, one optimizer step per call
(behaviour of `src/sharded_runtime/training/trainer.py:19-81`).

A step is three phases kept as separate methods: `_accumulate` runs the micro-batches and sums
their (already averaged) losses, `_checked_gradients` refuses missing or non-finite gradients
and returns them, and `train_step` applies the update and reports norms computed in float64.
"""

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
    squares = [torch.linalg.vector_norm(t.detach().double()) ** 2 for t in tensors]
    return float(torch.stack(squares).sum().sqrt()) if squares else 0.0


class Trainer:
    def __init__(self, model: nn.Module, lr: float, accumulation_steps: int = 1, *, tp_plan=None):
        if type(accumulation_steps) is not int or accumulation_steps <= 0:
            raise ValueError("accumulation_steps must be a positive integer")
        if tp_plan is not None and tp_plan.model is not model:
            raise ValueError("TP plan belongs to a different model")
        if getattr(model, "_tp_plan", None) is not tp_plan:
            raise ValueError("A converted model must be trained with its own TP/SP plan")
        self.model, self.tp_plan = model, tp_plan
        self.accumulation_steps, self.step_id = accumulation_steps, 0
        self.optimizer = torch.optim.SGD(model.parameters(), lr=lr)

    # ------------------------------------------------------------------ phases of a step
    def _micro_loss(self, output: Tensor) -> Tensor:
        plan = self.tp_plan
        loss = output.square().mean() if plan is None else plan.backward_loss(output)
        return loss / self.accumulation_steps

    def _accumulate(self, batch: Tensor) -> Tensor:
        running = batch.new_zeros(())
        for micro in batch.chunk(self.accumulation_steps, dim=0):
            loss = self._micro_loss(self.model(micro))
            if not torch.isfinite(loss):
                raise FloatingPointError(f"Non-finite loss at step {self.step_id}")
            loss.backward()
            running += loss.detach()
        if self.tp_plan is None:
            return running
        self.tp_plan.finalize_gradients()
        return self.tp_plan.reported_loss(running)

    def _checked_gradients(self) -> list[Tensor]:
        gradients = []
        for name, parameter in self.model.named_parameters():
            if parameter.grad is None:
                raise RuntimeError(f"Missing gradient for {name} at step {self.step_id}")
            if not torch.isfinite(parameter.grad).all():
                raise FloatingPointError(f"Non-finite gradient for {name} at step {self.step_id}")
            gradients.append(parameter.grad)
        return gradients

    # ------------------------------------------------------------------ public
    def train_step(self, batch: Tensor) -> StepResult:
        if batch.ndim != 3 or batch.shape[0] == 0 or batch.shape[0] % self.accumulation_steps:
            raise ValueError("Batch must be [B,S,H] with B divisible by accumulation_steps")
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        loss = self._accumulate(batch)
        gradient_l2 = l2_norm(self._checked_gradients())   # read before the update frees nothing
        self.optimizer.step()
        result = StepResult(self.step_id, loss.item(), gradient_l2, l2_norm(self.model.parameters()))
        self.step_id += 1
        return result


class ReferenceTrainer(Trainer):
    """Name kept for the unpartitioned reference path."""
