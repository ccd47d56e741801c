"""`WorkerSession`: the context manager every entry point runs inside.

What a worker needs before it can train is acquired in a fixed order -- the torchrun
environment, the rank log, a config validated for the execution mode, the NCCL launch-order
contract when the NCCL path runs `stream_ordered`, the process groups, the metadata dump -- and
released in the reverse order on every exit path: groups first (never with a barrier), log last.
The acquisitions are pushed on an `ExitStack` as they succeed, so a failure half-way releases
exactly what exists, logs "Worker bootstrap failed" on this rank and re-raises
(behaviour of `src/sharded_runtime/launch/bootstrap.py:11-74`).
"""

from __future__ import annotations

import logging
from contextlib import ExitStack
from pathlib import Path

from shardtrain_b200.config import Config, ConfigError
from shardtrain_b200.distributed.context import DistributedContext, WorkerEnvironment
from shardtrain_b200.distributed.nccl_ordering import prepare_nccl_launch_order
from shardtrain_b200.observability.logging import close_logger, make_rank_logger
from shardtrain_b200.observability.metadata import save_metadata

_LEVELS = {"DEBUG", "INFO", "WARNING", "ERROR"}


class WorkerSession:
    def __init__(self, config: Config, mode: str) -> None:
        if not config.debug.output_dir.strip():
            raise ConfigError("debug.output_dir must not be empty")
        self.config, self.mode = config, mode
        self.directory = Path(config.debug.output_dir)
        self.context: DistributedContext | None = None
        self.logger: logging.Logger | None = None
        self.worker: WorkerEnvironment | None = None
        self._resources: ExitStack | None = None

    # ------------------------------------------------------------------ acquisition steps
    @property
    def _log_level(self) -> str:
        level = self.config.debug.log_level
        return level if level in _LEVELS else "INFO"

    def _read_launcher_environment(self) -> WorkerEnvironment:
        try:
            return WorkerEnvironment.read()
        except ConfigError:
            # a malformed launcher environment has no rank yet: leave a rank-0 log behind
            orphan = make_rank_logger(self.directory, 0, self._log_level)
            orphan.exception("Worker environment validation failed")
            close_logger(orphan)
            raise

    def _wants_nccl_launch_order(self) -> bool:
        cfg, worker = self.config, self.worker
        return (worker.launched and worker.world_size > 1 and cfg.parallel.backend == "nccl"
                and cfg.runtime.communication_policy == "stream_ordered")

    def _log_if_bootstrap_failed(self, exc_type, exc, tb) -> bool:
        if exc_type is not None:
            self.logger.error("Worker bootstrap failed", exc_info=(exc_type, exc, tb))
        return False

    def __enter__(self) -> "WorkerSession":
        self.worker = self._read_launcher_environment()
        with ExitStack() as stack:
            self.logger = make_rank_logger(self.directory, self.worker.rank, self._log_level)
            stack.callback(close_logger, self.logger)
            stack.push(self._log_if_bootstrap_failed)      # runs before the log is closed
            cfg = self.config
            cfg.validate(self.worker.world_size, mode=self.mode)
            if self._wants_nccl_launch_order():
                prepare_nccl_launch_order()
                self.logger.info("NCCL host launch ordering armed")
            self.context = DistributedContext(cfg.parallel, self.worker,
                                              cfg.debug.distributed_timeout_seconds, self.logger)
            stack.callback(self.context.close)             # groups go before the log
            save_metadata(self.directory, cfg, self.worker, self.context.device)
            self.logger.info("Resolved config: %s", cfg.to_dict())
            # everything succeeded: keep the resources for __exit__ (the failure logger is not
            # part of a healthy session's teardown)
            kept = ExitStack()
            kept.callback(close_logger, self.logger)
            kept.callback(self.context.close)
            stack.pop_all()
            self._resources = kept
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if exc_type is not None:
            self.logger.error("Worker failed", exc_info=(exc_type, exc, tb))
        resources, self._resources = self._resources, None
        context = self.context
        try:
            if context is not None:
                context.close()
                if exc_type is None and context.cleanup_errors:
                    raise RuntimeError("Worker cleanup failed: " + "; ".join(context.cleanup_errors))
        finally:
            if resources is not None:
                resources.close()          # context.close() is idempotent; the log closes last
