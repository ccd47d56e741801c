"""Run metadata written next to the logs: resolved config and an environment snapshot per rank
(`resolved_config.rank{r}.yaml`, `environment.rank{r}.json`; reference:
`src/sharded_runtime/observability/metadata.py:16-60`)."""

from __future__ import annotations

import importlib.metadata
import json
import platform
import subprocess
import sys
from pathlib import Path
from typing import Any

import torch
import yaml


def git_revision() -> str | None:
    try:
        done = subprocess.run(
            ["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5, check=False
        )
    except (OSError, subprocess.TimeoutExpired):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def write_json(filename: Path, data: Any) -> None:
    # values json does not know (dtypes, paths, devices) are written as their text form
    text = json.dumps(data, indent=2, ensure_ascii=False, default=str)
    Path(filename).write_text(text + "\n", encoding="utf-8")


def _version(package: str) -> str | None:
    try:
        return importlib.metadata.version(package)
    except importlib.metadata.PackageNotFoundError:
        return None


def environment_snapshot(worker, device: torch.device) -> dict[str, Any]:
    from shardtrain_b200 import ops

    cuda = device.type == "cuda"
    return {
        "python": sys.version,
        "executable": sys.executable,
        "platform": platform.platform(),
        "torch": torch.__version__,
        "packages": {name: _version(name) for name in ("torch", "PyYAML")},
        "cuda_build": torch.version.cuda,
        "nccl_available": torch.distributed.is_nccl_available(),
        "gloo_available": torch.distributed.is_gloo_available(),
        "device": str(device),
        "device_name": torch.cuda.get_device_name(device) if cuda else "CPU",
        "sm_100a_extension": ops.extension_path(),
        "rank": worker.rank,
        "local_rank": worker.local_rank,
        "world_size": worker.world_size,
        "git_commit": git_revision(),
    }


def save_metadata(directory: Path, config, worker, device: torch.device) -> None:
    directory = Path(directory)
    (directory / f"resolved_config.rank{worker.rank}.yaml").write_text(
        yaml.safe_dump(config.to_dict(), sort_keys=False), encoding="utf-8"
    )
    write_json(directory / f"environment.rank{worker.rank}.json", environment_snapshot(worker, device))
