"""Per-rank JSON-lines logging.

Every rank writes `rank{r}.jsonl` in the run directory; rank 0 also mirrors its level to stderr
while the other ranks only surface errors there (artifact names follow the reference,
`src/sharded_runtime/observability/logging.py:8-44`).

One handler, `RankSink`, owns both destinations: it renders a record once as a JSON row for the
file and, when the record passes the console threshold of this rank, once as a short text line.
"""

from __future__ import annotations

import json
import logging
import sys
import traceback
from datetime import datetime, timezone
from pathlib import Path


class RankSink(logging.Handler):
    """File (every record, JSON lines) + stderr (from `console_level` up) for one rank."""

    def __init__(self, path: Path, rank: int, console_level: int) -> None:
        super().__init__()
        self.rank, self.console_level = rank, console_level
        self.file = open(path, "a", encoding="utf-8")

    def row(self, record: logging.LogRecord) -> dict:
        fields = {"time_utc": datetime.fromtimestamp(record.created, timezone.utc).isoformat(),
                  "rank": self.rank, "level": record.levelname, "message": record.getMessage()}
        if record.exc_info:
            fields["exception"] = "".join(traceback.format_exception(*record.exc_info)).rstrip()
        return fields

    def emit(self, record: logging.LogRecord) -> None:
        try:
            fields = self.row(record)
            self.file.write(json.dumps(fields, ensure_ascii=False) + "\n")
            self.file.flush()
            if record.levelno >= self.console_level:
                text = f"[rank {self.rank}] {fields['level']} {fields['message']}"
                if "exception" in fields:
                    text += "\n" + fields["exception"]
                print(text, file=sys.stderr, flush=True)
        except Exception:  # noqa: BLE001 - logging must never take the run down
            self.handleError(record)

    def close(self) -> None:
        try:
            self.file.close()
        finally:
            super().close()


def close_logger(logger: logging.Logger) -> None:
    while logger.handlers:
        handler = logger.handlers[0]
        logger.removeHandler(handler)
        handler.close()


def make_rank_logger(directory: Path, rank: int, level: str = "INFO") -> logging.Logger:
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    logger = logging.getLogger(f"shardtrain.rank{rank}")
    close_logger(logger)                       # a re-created logger must not write twice
    logger.setLevel(level)
    logger.propagate = False
    console = logging.getLevelName(level) if rank == 0 else logging.ERROR
    logger.addHandler(RankSink(directory / f"rank{rank}.jsonl", rank, console))
    return logger
