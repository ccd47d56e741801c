"""Optional capture around the training window: torch profiler trace or NVTX emission for an
external Nsight session, plus allocator history snapshots and per-step memory rows.

Modes and artifact names (`profile.rank{r}.json`, `memory.{start,end}.rank{r}.pickle`,
`profiling.rank{r}.json`) follow `src/sharded_runtime/observability/profiling.py:11-127`.
Numbers taken while a capture is active are never reported as throughput.
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

from shardtrain_b200.observability.metadata import write_json

NVTX_ENV = "SHARDTRAIN_NVTX"


class ProfileCapture:
    def __init__(self, directory, rank, device, *, mode="torch", max_entries=200_000,
                 detail="low_overhead"):
        if mode not in {"torch", "nsight", "off"}:
            raise ValueError("Unknown profile mode")
        if detail not in {"low_overhead", "full"}:
            raise ValueError("Unknown profile detail")
        self.directory, self.rank = Path(directory), rank
        self.device = torch.device(device)
        self.mode, self.detail, self.max_entries = mode, detail, max_entries
        self.rows: list[dict] = []
        self._profiler = None
        self._nvtx = None
        self._history_on = False
        self._saved_env: str | None = None

    @property
    def _cuda(self) -> bool:
        return self.device.type == "cuda"

    def start(self) -> None:
        if self.mode == "off":
            return
        self.directory.mkdir(parents=True, exist_ok=True)
        activities = [torch.profiler.ProfilerActivity.CPU]
        if self._cuda:
            full = self.detail == "full"
            torch.cuda.memory._record_memory_history(
                context="all" if full else "alloc",
                stacks="all" if full else "python",
                max_entries=self.max_entries,
            )
            self._history_on = True
            torch.cuda.memory._dump_snapshot(str(self.directory / f"memory.start.rank{self.rank}.pickle"))
            activities.append(torch.profiler.ProfilerActivity.CUDA)
            self._saved_env = os.environ.get(NVTX_ENV)
            os.environ[NVTX_ENV] = "1"
        if self.mode == "torch":
            # no shape recording: it can keep tensors alive and disturb reshard lifetime checks
            self._profiler = torch.profiler.profile(
                activities=activities, record_shapes=False, profile_memory=True,
                with_stack=self.detail == "full",
            )
            self._profiler.start()
        elif self._cuda:
            self._nvtx = torch.autograd.profiler.emit_nvtx(record_shapes=self.detail == "full")
            self._nvtx.__enter__()

    def step(self, step: int) -> None:
        if self._cuda and self.mode != "off":
            self.rows.append(
                {
                    "step": step,
                    "allocated": torch.cuda.memory_allocated(self.device),
                    "reserved": torch.cuda.memory_reserved(self.device),
                    "max_allocated": torch.cuda.max_memory_allocated(self.device),
                    "max_reserved": torch.cuda.max_memory_reserved(self.device),
                }
            )
            torch.cuda.nvtx.mark(f"shardtrain/step_complete/{step}/rank{self.rank}")
        if self._profiler is not None:
            self._profiler.step()

    def close(self) -> None:
        if self.mode == "off":
            return
        errors: list[str] = []
        try:
            if self._profiler is not None:
                self._profiler.stop()
                self._profiler.export_chrome_trace(str(self.directory / f"profile.rank{self.rank}.json"))
            if self._nvtx is not None:
                self._nvtx.__exit__(None, None, None)
        except Exception as exc:  # noqa: BLE001
            errors.append(repr(exc))
        if self._history_on:
            try:
                torch.cuda.memory._dump_snapshot(str(self.directory / f"memory.end.rank{self.rank}.pickle"))
            except Exception as exc:  # noqa: BLE001
                errors.append(repr(exc))
            torch.cuda.memory._record_memory_history(enabled=None)
            if self._saved_env is None:
                os.environ.pop(NVTX_ENV, None)
            else:
                os.environ[NVTX_ENV] = self._saved_env
            self._history_on = False
        write_json(
            self.directory / f"profiling.rank{self.rank}.json",
            {
                "mode": self.mode,
                "rank": self.rank,
                "device": str(self.device),
                "profile_detail": self.detail,
                "memory_history_max_entries": self.max_entries,
                "memory": self.rows,
                "errors": errors,
                "note": "allocator snapshots exclude peer-memory arenas allocated with cudaMalloc",
            },
        )
        if errors:
            raise RuntimeError(f"Failed to save profiling artifacts: {errors}")
