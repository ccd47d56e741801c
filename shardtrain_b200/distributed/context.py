"""Process-group ownership for one worker: the default group, four role communicators, device
binding, and a teardown that never waits for a peer.

Behaviour kept from the reference's `DistributedContext`
(`src/sharded_runtime/distributed/context.py:45-211`): the context must create the default group
itself, every rank creates every communicator in `Topology.creation_order` (creation is
collective), close callbacks run before any group is destroyed, and cleanup issues no barrier
(after a failure some peer may never arrive).  The teardown is a list of labelled steps; each
step's failure is logged and collected in `cleanup_errors` without stopping the later steps.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from datetime import timedelta
from typing import Any, Callable, Mapping

import torch
import torch.distributed as dist

from shardtrain_b200.config import ConfigError, ParallelConfig
from shardtrain_b200.distributed.topology import GROUP_ROLES, Topology

_LAUNCHER_VARIABLES = ("RANK", "LOCAL_RANK", "WORLD_SIZE")


@dataclass(frozen=True)
class WorkerEnvironment:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    launched: bool = False

    @classmethod
    def read(cls, environ: Mapping[str, str] | None = None) -> "WorkerEnvironment":
        """The torchrun variables: all three or none (a plain single-process run)."""
        env = os.environ if environ is None else environ
        present = [name for name in _LAUNCHER_VARIABLES if name in env]
        if not present:
            return cls()
        if len(present) != len(_LAUNCHER_VARIABLES):
            raise ConfigError("torchrun requires RANK, LOCAL_RANK and WORLD_SIZE together")
        try:
            rank, local_rank, world = (int(env[name]) for name in _LAUNCHER_VARIABLES)
        except ValueError as exc:
            raise ConfigError("torchrun rank environment values must be integers") from exc
        if world <= 0 or not 0 <= rank < world or local_rank < 0:
            raise ConfigError("Invalid RANK/LOCAL_RANK/WORLD_SIZE in worker environment")
        return cls(rank, local_rank, world, True)


def _backend_problem(backend: str) -> str | None:
    """Why this PyTorch build cannot serve `backend` (None: it can)."""
    if not os.environ.get("MASTER_ADDR") or not os.environ.get("MASTER_PORT"):
        return "torchrun launch requires MASTER_ADDR and MASTER_PORT"
    if not dist.is_available():
        return "This PyTorch build does not support torch.distributed"
    available = {"nccl": dist.is_nccl_available, "gloo": dist.is_gloo_available}.get(backend)
    if available is not None and not available():
        return f"{'NCCL' if backend == 'nccl' else 'Gloo'} is unavailable in this PyTorch build"
    return None


class DistributedContext:
    def __init__(self, parallel: ParallelConfig, worker: WorkerEnvironment, timeout_seconds: int,
                 logger: logging.Logger) -> None:
        self.logger, self.parallel, self.worker = logger, parallel, worker
        self.topology = Topology(parallel.fsdp_degree, parallel.tp_degree)
        if self.topology.world_size != worker.world_size:
            raise ConfigError("Worker world size does not match topology")
        self.coordinate = self.topology.coordinate(worker.rank)
        self.device = torch.device("cpu")
        self.cleanup_errors: list[str] = []
        self._callbacks: list[Callable[[], None]] = []
        self._groups: list[Any] = []          # the role communicators this rank belongs to
        self._owns_default = False
        self._closed = False
        self._forget_groups()
        try:
            self.device = self._bound_device()
            if dist.is_initialized():
                raise RuntimeError("DistributedContext requires ownership of an uninitialized group")
            if worker.launched:
                self._create_groups(timedelta(seconds=timeout_seconds))
        except BaseException:
            self.close()
            raise
        logger.info("Context ready: rank=%d local_rank=%d coordinate=%s device=%s groups=%s",
                    worker.rank, worker.local_rank, self.coordinate, self.device,
                    self.topology.groups_for_rank(worker.rank))

    # ------------------------------------------------------------------ setup
    def _forget_groups(self) -> None:
        for role in GROUP_ROLES:
            setattr(self, f"{role}_group", None)

    def _bound_device(self) -> torch.device:
        if self.parallel.device != "cuda":
            return torch.device("cpu")
        if not torch.cuda.is_available():
            raise ConfigError("CUDA was requested but is unavailable")
        index = self.worker.local_rank
        if index >= torch.cuda.device_count():
            raise ConfigError("LOCAL_RANK exceeds the number of visible CUDA devices")
        torch.cuda.set_device(index)
        return torch.device("cuda", index)

    def _create_groups(self, timeout: timedelta) -> None:
        backend = self.parallel.backend
        problem = _backend_problem(backend)
        if problem is not None:
            raise ConfigError(problem)
        options = {"device_id": self.device} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, rank=self.worker.rank,
                                world_size=self.worker.world_size, timeout=timeout, **options)
        self._owns_default = True
        # group creation is collective over the default group: every rank walks the whole list
        for role, members in self.topology.creation_order:
            self.logger.debug("Creating %s group ranks=%s", role, members)
            group = dist.new_group(ranks=list(members), backend=backend, timeout=timeout)
            if self.worker.rank in members:
                self._groups.append(group)
                setattr(self, f"{role}_group", group)

    # ------------------------------------------------------------------ use
    @property
    def sp_group(self) -> Any:
        """Sequence parallelism shares the TP communicator; it is not a mesh dimension."""
        return self.tp_group

    def smoke_collectives(self) -> dict[str, dict[str, Any]]:
        """One all_gather + all_reduce per role communicator, checked against rank arithmetic."""
        if self._closed:
            raise RuntimeError("Cannot use a closed DistributedContext")
        report = {}
        for role, members in self.topology.groups_for_rank(self.worker.rank).items():
            token = torch.tensor([float(self.worker.rank + 1)], device=self.device)
            seen = [torch.empty_like(token) for _ in members]
            if self._owns_default:
                group = getattr(self, f"{role}_group")
                dist.all_gather(seen, token, group=group)
                dist.all_reduce(token, op=dist.ReduceOp.SUM, group=group)
            else:
                seen[0].copy_(token)
            total, gathered = token.item(), [t.item() for t in seen]
            expected = [float(r + 1) for r in members]
            if total != sum(expected) or gathered != expected:
                raise AssertionError(f"{role} collective mismatch: {total}, {gathered}")
            report[role] = {"ranks": list(members), "sum": total, "gather": gathered}
        self.logger.info("Collective smoke passed: %s", report)
        return report

    def add_close_callback(self, callback: Callable[[], None]) -> None:
        """Local cleanup (e.g. flushing event logs) run once before the groups are destroyed."""
        if self._closed:
            raise RuntimeError("Cannot register cleanup on a closed DistributedContext")
        if not callable(callback):
            raise TypeError("DistributedContext close callback must be callable")
        self._callbacks.append(callback)

    # ------------------------------------------------------------------ teardown
    def _teardown_steps(self):
        """(label, log message, action) in execution order.  No step waits for a peer."""
        for index, callback in enumerate(self._callbacks):
            yield (f"close callback {index}", f"Failed to run local close callback {index}", callback)
        for group in reversed(self._groups):
            yield ("destroy subgroup", "Failed to destroy subgroup",
                   lambda group=group: dist.destroy_process_group(group))
        if self._owns_default:
            yield ("destroy default group", "Failed to destroy default process group",
                   dist.destroy_process_group)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        steps = list(self._teardown_steps())
        self._callbacks = []
        for label, message, action in steps:
            try:
                action()
            except Exception as exc:  # noqa: BLE001 - collected; later steps still run
                self.cleanup_errors.append(f"{label}: {exc!r}")
                self.logger.exception(message)
        self._groups.clear()
        self._owns_default = False
        self._forget_groups()
        self.logger.info("Context closed")

    def __enter__(self) -> "DistributedContext":
        return self

    def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
        self.close()
        if exc_type is None and self.cleanup_errors:
            raise RuntimeError("DistributedContext cleanup failed: " + "; ".join(self.cleanup_errors))
