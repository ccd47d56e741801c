"""Contract for the NCCL baseline path's `stream_ordered` policy.

Host-order-only submission of collectives on several streams relies on NCCL's implicit launch
ordering: NCCL >= 2.26, CUDA build/runtime/driver >= 12.3 and `NCCL_LAUNCH_ORDER_IMPLICIT=1`
set before any communicator exists (reference: `src/sharded_runtime/distributed/nccl_ordering.py:11-79`).
The peer-memory backend does not need it: its kernels order themselves with flags in peer memory.
"""

from __future__ import annotations

import ctypes
import os

ENV_NAME = "NCCL_LAUNCH_ORDER_IMPLICIT"
MIN_NCCL = (2, 26)
MIN_CUDA = 12030


def _cuda_versions() -> dict[str, int | None]:
    found: dict[str, int | None] = {"runtime": None, "driver": None}
    for name in ("libcudart.so", "libcudart.so.12", "libcudart.so.13"):
        try:
            lib = ctypes.CDLL(name)
        except OSError:
            continue
        value = ctypes.c_int(0)
        if lib.cudaRuntimeGetVersion(ctypes.byref(value)) == 0:
            found["runtime"] = value.value
        value = ctypes.c_int(0)
        if lib.cudaDriverGetVersion(ctypes.byref(value)) == 0:
            found["driver"] = value.value
        break
    return found


def launch_order_facts() -> dict:
    import torch

    build = torch.version.cuda
    build_code = None
    if build:
        major, minor = (int(x) for x in build.split(".")[:2])
        build_code = major * 1000 + minor * 10
    nccl = None
    try:
        nccl = tuple(torch.cuda.nccl.version())
    except Exception:  # noqa: BLE001 - CPU-only builds have no NCCL
        pass
    facts = {
        "env": os.environ.get(ENV_NAME),
        "nccl_version": list(nccl) if nccl else None,
        "cuda_build": build_code,
        **{f"cuda_{k}": v for k, v in _cuda_versions().items()},
    }
    facts["satisfied"] = bool(
        facts["env"] == "1"
        and nccl is not None
        and tuple(nccl[:2]) >= MIN_NCCL
        and all((facts[k] or 0) >= MIN_CUDA for k in ("cuda_build", "cuda_runtime", "cuda_driver"))
    )
    return facts


def prepare_nccl_launch_order() -> None:
    """Set the variable; must run before the first communicator is created."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        raise RuntimeError(f"{ENV_NAME} must be set before process-group creation")
    current = os.environ.get(ENV_NAME)
    if current not in (None, "1"):
        raise RuntimeError(f"{ENV_NAME}={current!r} conflicts with communication_policy=stream_ordered")
    os.environ[ENV_NAME] = "1"


def require_nccl_launch_order() -> dict:
    facts = launch_order_facts()
    if not facts["satisfied"]:
        raise RuntimeError(f"NCCL implicit launch order is unavailable: {facts}")
    return facts
