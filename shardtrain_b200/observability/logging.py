"""Per-rank JSON-lines logging.

Every rank writes `rank{r}.jsonl` in the run directory; rank 0 also mirrors its level to stderr
while the other ranks only surface errors there (artifact names follow the reference,
`src/sharded_runtime/observability/logging.py:8-44`).
"""

from __future__ import annotations

import json
import logging
import sys
from datetime import datetime, timezone
from pathlib import Path


class RankJsonFormatter(logging.Formatter):
    def __init__(self, rank: int) -> None:
        super().__init__()
        self.rank = rank

    def format(self, record: logging.LogRecord) -> str:
        row = {
            "time_utc": datetime.fromtimestamp(record.created, timezone.utc).isoformat(),
            "rank": self.rank,
            "level": record.levelname,
            "message": record.getMessage(),
        }
        if record.exc_info:
            row["exception"] = self.formatException(record.exc_info)
        return json.dumps(row, ensure_ascii=False)


def close_logger(logger: logging.Logger) -> None:
    for handler in list(logger.handlers):
        handler.close()
        logger.removeHandler(handler)


def make_rank_logger(directory: Path, rank: int, level: str = "INFO") -> logging.Logger:
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    logger = logging.getLogger(f"shardtrain.rank{rank}")
    close_logger(logger)
    logger.setLevel(level)
    logger.propagate = False
    to_file = logging.FileHandler(directory / f"rank{rank}.jsonl", encoding="utf-8")
    to_file.setFormatter(RankJsonFormatter(rank))
    to_console = logging.StreamHandler(sys.stderr)
    to_console.setLevel(level if rank == 0 else logging.ERROR)
    to_console.setFormatter(logging.Formatter(f"[rank {rank}] %(levelname)s %(message)s"))
    logger.addHandler(to_file)
    logger.addHandler(to_console)
    return logger
