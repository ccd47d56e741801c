"""SGD trainer over the sharded runtime for the toy block model: owns data, loss and optimizer;
materialisation and buffers stay inside the runtime
(`src/sharded_runtime/training/sharded_trainer.py:8-46`)."""

from __future__ import annotations

from shardtrain_b200.training.optim import ArenaSGD
from shardtrain_b200.training.trainer import StepResult, l2_norm


class ShardedTrainer:
    def __init__(self, model, runtime, lr):
        self.model, self.runtime = model, runtime
        self.optimizer = ArenaSGD(runtime, lr=lr)
        runtime.bind_optimizer(self.optimizer)
        self.step_id = 0

    def train_step(self, batch, target):
        runtime = self.runtime
        with runtime.compute_context():
            try:
                runtime.begin_step(self.step_id)
                runtime.zero_grad()
                loss = runtime.local_loss(self.model(batch), target)
                loss.backward()
                runtime.finalize_backward()
                reported = runtime.reported_loss(loss)
                grad_l2 = l2_norm(p.grad for p in runtime.sharded_parameters())
                self.optimizer.step()
                param_l2 = l2_norm(runtime.sharded_parameters())
                runtime.end_step()
                result = StepResult(self.step_id, reported.item(), grad_l2, param_l2)
                self.step_id += 1
                return result
            except BaseException as exc:
                runtime.fail(exc)
                raise
