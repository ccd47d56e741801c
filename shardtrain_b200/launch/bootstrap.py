"""`WorkerSession`: the context manager every entry point runs inside.

Order on entry: read the torchrun environment, open the rank log, validate the config for the
execution mode, arm the NCCL launch-order contract when the NCCL path runs `stream_ordered`,
create the process groups, dump metadata.  Every exit path closes the groups (without a barrier)
and the log (reference: `src/sharded_runtime/launch/bootstrap.py:11-74`).
"""

from __future__ import annotations

import logging
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

    def __enter__(self) -> "WorkerSession":
        cfg = self.config
        level = cfg.debug.log_level if cfg.debug.log_level in _LEVELS else "INFO"
        try:
            self.worker = WorkerEnvironment.read()
        except ConfigError:
            # even a malformed launcher environment leaves a log behind
            logger = make_rank_logger(self.directory, 0, level)
            logger.exception("Worker environment validation failed")
            close_logger(logger)
            raise
        self.logger = make_rank_logger(self.directory, self.worker.rank, level)
        try:
            cfg.validate(self.worker.world_size, mode=self.mode)
            nccl_ordered = (
                self.worker.launched
                and self.worker.world_size > 1
                and cfg.parallel.backend == "nccl"
                and cfg.runtime.communication_policy == "stream_ordered"
            )
            if nccl_ordered:
                prepare_nccl_launch_order()
                self.logger.info("NCCL host launch ordering armed")
            self.context = DistributedContext(
                cfg.parallel, self.worker, cfg.debug.distributed_timeout_seconds, self.logger
            )
            save_metadata(self.directory, cfg, self.worker, self.context.device)
            self.logger.info("Resolved config: %s", cfg.to_dict())
            return self
        except BaseException:
            self.logger.exception("Worker bootstrap failed")
            if self.context is not None:
                self.context.close()
            close_logger(self.logger)
            raise

    def __exit__(self, exc_type, exc, tb) -> None:
        try:
            if exc_type is not None:
                self.logger.error("Worker failed", exc_info=(exc_type, exc, tb))
            if self.context is not None:
                self.context.close()
                if exc_type is None and self.context.cleanup_errors:
                    raise RuntimeError(
                        "Worker cleanup failed: " + "; ".join(self.context.cleanup_errors)
                    )
        finally:
            if self.logger is not None:
                close_logger(self.logger)
