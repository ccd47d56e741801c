"""SGD trainer over the sharded runtime for the toy block model: owns data, loss and optimizer;
materialisation and buffers stay inside the runtime
(`src/sharded_runtime/training/sharded_trainer.py:8-46`).

The step protocol (`begin_step` -> forward -> backward -> `finalize_backward` -> optimizer ->
`end_step`, any exception marks the runtime FAILED) is written once as a context manager,
`guarded_step`, with the three phases of a step as its body.
"""

from __future__ import annotations

from contextlib import contextmanager

from shardtrain_b200.training.optim import ArenaSGD
from shardtrain_b200.training.trainer import StepResult, l2_norm


@contextmanager
def guarded_step(runtime, step_id):
    """One optimizer step on the runtime's compute stream.  The body runs between `begin_step`
    and `end_step`; whatever it raises leaves the runtime FAILED before it propagates."""
    with runtime.compute_context():
        try:
            runtime.begin_step(step_id)
            yield
            runtime.end_step()
        except BaseException as failure:
            runtime.fail(failure)
            raise


class ShardedTrainer:
    def __init__(self, model, runtime, lr):
        self.model, self.runtime = model, runtime
        self.optimizer = ArenaSGD(runtime, lr=lr)
        runtime.bind_optimizer(self.optimizer)
        self.step_id = 0

    def _gradients(self, batch, target):
        """Forward, loss, backward and the optimizer boundary; returns the loss to report."""
        runtime = self.runtime
        runtime.zero_grad()
        loss = runtime.local_loss(self.model(batch), target)
        loss.backward()
        runtime.finalize_backward()
        return runtime.reported_loss(loss)

    def train_step(self, batch, target):
        runtime = self.runtime
        with guarded_step(runtime, self.step_id):
            reported = self._gradients(batch, target)
            norms = [l2_norm(p.grad for p in runtime.sharded_parameters())]
            self.optimizer.step()
            norms.append(l2_norm(runtime.sharded_parameters()))
        result = StepResult(self.step_id, reported.item(), *norms)
        self.step_id += 1
        return result
