"""Optimizers over the flat shard arena.

`ArenaAdamW` / `ArenaSGD` are `torch.optim.Optimizer`s whose `param_groups` hold exactly the
runtime's shard leaves (so the runtime's ownership checks and hooks apply unchanged), but whose
state is one flat `exp_avg` / `exp_avg_sq` arena and whose `step()` is a single kernel launch over
every leaf on sm_100a (a few whole-arena tensor ops on CPU) instead of one launch set per leaf as
in `torch.optim.AdamW(foreach=False)` (`src/sharded_runtime/training/qwen2_trainer.py:48`).
When `fuse_into_reduction` is set, the last micro-step's reduce-scatter kernel applies the update
to each unit as its gradients land, and `step()` only updates what was not covered.
"""

from __future__ import annotations

import torch


class _ArenaOptimizer(torch.optim.Optimizer):
    def __init__(self, runtime, defaults):
        self.runtime = runtime
        super().__init__(runtime.sharded_parameters(), defaults)
        self.arena_step = 0
        self.units_updated: set[int] = set()
        self.fuse_into_reduction = False
        # True after a step in which every unit was updated by the fused reduce-scatter kernel,
        # which writes the compute-dtype shadow of the shards next to the FP32 masters
        self.shadow_current = False

    @property
    def _ops(self):
        return self.runtime.fused.ops if self.runtime.fused is not None else None

    def _pending_ranges(self):
        """Arena ranges of the units that the fused reduction has not already updated."""
        plan = self.runtime.plan
        todo = [plan.unit_ranges[u.unit_id] for u in self.runtime.units
                if u.unit_id not in self.units_updated]
        merged = []
        for lo, hi in sorted(todo):
            if merged and lo <= merged[-1][1] + 4:
                merged[-1] = (merged[-1][0], hi)
            else:
                merged.append((lo, hi))
        return merged


class ArenaAdamW(_ArenaOptimizer):
    def __init__(self, runtime, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        super().__init__(runtime, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        total = runtime.param_arena.numel()
        make = runtime.fused.state_arena if runtime.fused is not None else (
            lambda tag: torch.zeros(total, dtype=torch.float32, device=runtime.device))
        self.exp_avg, self.exp_avg_sq = make("exp_avg"), make("exp_avg_sq")
        for h in runtime.registry.values():
            q = h.spec.fsdp_shard_numel
            self.state[h.local_shard] = {
                "step": torch.tensor(0.0),
                "exp_avg": self.exp_avg.narrow(0, h.arena_offset, q),
                "exp_avg_sq": self.exp_avg_sq.narrow(0, h.arena_offset, q),
            }

    def kernel_args(self, step=None):
        g = self.param_groups[0]
        t = self.arena_step + 1 if step is None else step
        b1, b2 = g["betas"]
        return (g["lr"], b1, b2, g["eps"], g["weight_decay"], 1 - b1 ** t, 1 - b2 ** t, 1.0)

    @torch.no_grad()
    def step(self, closure=None):
        rt = self.runtime
        args = self.kernel_args()
        pending = self._pending_ranges()
        self.shadow_current = not pending and rt.fused is not None
        for lo, hi in pending:
            p, g = rt.param_arena[lo:hi], rt.grad_arena[lo:hi]
            m, v = self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi]
            if self._ops is not None:
                self._ops.adamw(p, g, m, v, *args)
            else:
                lr, b1, b2, eps, wd, bc1, bc2, _ = args
                p.mul_(1 - lr * wd)
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                p.addcdiv_(m, (v.sqrt() / bc2 ** 0.5).add_(eps), value=-lr / bc1)
        self.arena_step += 1
        self.units_updated.clear()
        for state in self.state.values():
            state["step"] += 1


class ArenaSGD(_ArenaOptimizer):
    def __init__(self, runtime, lr=1e-3):
        super().__init__(runtime, dict(lr=lr))

    @torch.no_grad()
    def step(self, closure=None):
        rt = self.runtime
        lr = self.param_groups[0]["lr"]
        self.shadow_current = False
        if self._ops is not None:
            self._ops.sgd(rt.param_arena, rt.grad_arena, lr)
        else:
            rt.param_arena.add_(rt.grad_arena, alpha=-lr)
        self.arena_step += 1
