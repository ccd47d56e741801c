"""Process-group ownership for one worker: default group, four role communicators, device binding.

Mirrors the behaviour of the reference's `DistributedContext`
(`src/sharded_runtime/distributed/context.py:45-211`): the context must create the default group
itself, every rank creates every communicator in `Topology.creation_order`, close callbacks run
before destruction, and cleanup never issues a barrier (a missing peer must not hang it).
On CUDA it can additionally build the NVLink peer-memory tables used by the fused kernels
(`shardtrain_b200.distributed.peer`).
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


@dataclass(frozen=True)
class WorkerEnvironment:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    launched: bool = False

    @classmethod
    def read(cls, environ: Mapping[str, str] | None = None) -> "WorkerEnvironment":
        env = os.environ if environ is None else environ
        names = ("RANK", "LOCAL_RANK", "WORLD_SIZE")
        have = [n in env for n in names]
        if not any(have):
            return cls()
        if not all(have):
            raise ConfigError("torchrun requires RANK, LOCAL_RANK and WORLD_SIZE together")
        try:
            rank, local_rank, world = (int(env[n]) for n in names)
        except ValueError as exc:
            raise ConfigError("torchrun rank environment values must be integers") from exc
        if world <= 0 or not 0 <= rank < world or local_rank < 0:
            raise ConfigError("Invalid RANK/LOCAL_RANK/WORLD_SIZE in worker environment")
        return cls(rank, local_rank, world, True)


class DistributedContext:
    def __init__(
        self,
        parallel: ParallelConfig,
        worker: WorkerEnvironment,
        timeout_seconds: int,
        logger: logging.Logger,
    ) -> None:
        self.logger, self.parallel, self.worker = logger, parallel, worker
        self.topology = Topology(parallel.fsdp_degree, parallel.tp_degree)
        if self.topology.world_size != worker.world_size:
            raise ConfigError("Worker world size does not match topology")
        self.coordinate = self.topology.coordinate(worker.rank)
        self.device = torch.device("cpu")
        self.cleanup_errors: list[str] = []
        self._callbacks: list[Callable[[], None]] = []
        self._groups: list[Any] = []
        self._owns_default = False
        self._closed = False
        for role in GROUP_ROLES:
            setattr(self, f"{role}_group", None)
        try:
            self._bind_device()
            if dist.is_initialized():
                raise RuntimeError("DistributedContext requires ownership of an uninitialized group")
            if worker.launched:
                self._create_groups(timedelta(seconds=timeout_seconds))
            logger.info(
                "Context ready: rank=%d local_rank=%d coordinate=%s device=%s groups=%s",
                worker.rank, worker.local_rank, self.coordinate, self.device,
                self.topology.groups_for_rank(worker.rank),
            )
        except BaseException:
            self.close()
            raise

    # ------------------------------------------------------------------ setup
    def _bind_device(self) -> None:
        if self.parallel.device != "cuda":
            return
        if not torch.cuda.is_available():
            raise ConfigError("CUDA was requested but is unavailable")
        if self.worker.local_rank >= torch.cuda.device_count():
            raise ConfigError("LOCAL_RANK exceeds the number of visible CUDA devices")
        torch.cuda.set_device(self.worker.local_rank)
        self.device = torch.device("cuda", self.worker.local_rank)

    def _create_groups(self, timeout: timedelta) -> None:
        backend = self.parallel.backend
        if not os.environ.get("MASTER_ADDR") or not os.environ.get("MASTER_PORT"):
            raise ConfigError("torchrun launch requires MASTER_ADDR and MASTER_PORT")
        if not dist.is_available():
            raise ConfigError("This PyTorch build does not support torch.distributed")
        if backend == "nccl" and not dist.is_nccl_available():
            raise ConfigError("NCCL is unavailable in this PyTorch build")
        if backend == "gloo" and not dist.is_gloo_available():
            raise ConfigError("Gloo is unavailable in this PyTorch build")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = self.device
        dist.init_process_group(
            backend=backend, rank=self.worker.rank, world_size=self.worker.world_size,
            timeout=timeout, **kwargs,
        )
        self._owns_default = True
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
            mine = torch.tensor([float(self.worker.rank + 1)], device=self.device)
            parts = [torch.empty_like(mine) for _ in members]
            if self._owns_default:
                group = getattr(self, f"{role}_group")
                dist.all_gather(parts, mine, group=group)
                dist.all_reduce(mine, op=dist.ReduceOp.SUM, group=group)
            else:
                parts[0].copy_(mine)
            total, seen = mine.item(), [p.item() for p in parts]
            if total != sum(r + 1 for r in members) or seen != [float(r + 1) for r in members]:
                raise AssertionError(f"{role} collective mismatch: {total}, {seen}")
            report[role] = {"ranks": list(members), "sum": total, "gather": seen}
        self.logger.info("Collective smoke passed: %s", report)
        return report

    def add_close_callback(self, callback: Callable[[], None]) -> None:
        """Local cleanup (e.g. flushing event logs) run once before the groups are destroyed."""
        if self._closed:
            raise RuntimeError("Cannot register cleanup on a closed DistributedContext")
        if not callable(callback):
            raise TypeError("DistributedContext close callback must be callable")
        self._callbacks.append(callback)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        callbacks, self._callbacks = self._callbacks, []
        for index, callback in enumerate(callbacks):
            try:
                callback()
            except Exception as exc:  # noqa: BLE001
                self.cleanup_errors.append(f"close callback {index}: {exc!r}")
                self.logger.exception("Failed to run local close callback %d", index)
        # No barrier here: after a failure some peer may never arrive.
        for group in reversed(self._groups):
            try:
                dist.destroy_process_group(group)
            except Exception as exc:  # noqa: BLE001
                self.cleanup_errors.append(f"destroy subgroup: {exc!r}")
                self.logger.exception("Failed to destroy subgroup")
        self._groups.clear()
        if self._owns_default:
            try:
                dist.destroy_process_group()
            except Exception as exc:  # noqa: BLE001
                self.cleanup_errors.append(f"destroy default group: {exc!r}")
                self.logger.exception("Failed to destroy default process group")
            finally:
                self._owns_default = False
        for role in GROUP_ROLES:
            setattr(self, f"{role}_group", None)
        self.logger.info("Context closed")

    def __enter__(self) -> "DistributedContext":
        return self

    def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
        self.close()
        if exc_type is None and self.cleanup_errors:
            raise RuntimeError("DistributedContext cleanup failed: " + "; ".join(self.cleanup_errors))
