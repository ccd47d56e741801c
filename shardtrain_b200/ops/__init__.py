"""Python side of the sm_100a extension.

`load()` returns `torch.ops.stb` after loading the in-tree `_C.so`.  On a machine with a GPU the
extension is mandatory: a missing or unloadable library raises instead of falling back to
PyTorch ops.  On a machine without CUDA `available()` is False and the portable (CPU/gloo)
executor is used.
"""

from __future__ import annotations

from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent.parent / "_C.so"
_loaded = False


def extension_path() -> str | None:
    return str(_LIB) if _LIB.exists() else None


def available() -> bool:
    return torch.cuda.is_available()


class LaunchCounter:
    """Reads the extension's own launch counter: every kernel launch site of the library counts
    itself, so `launches` is the exact number of this package's kernels launched by this process."""

    @property
    def launches(self) -> int:
        return int(_load_namespace().launch_count())


def enable_launch_counting():
    """Counter whose `launches` attribute benchmarks read before and after their timed region."""
    return LaunchCounter()


def load():
    return _load_namespace()


def _load_namespace():
    global _loaded
    if not _loaded:
        if not _LIB.exists():
            raise RuntimeError(
                f"{_LIB} is missing: build it with `python -m shardtrain_b200.build_ext` "
                "(the CUDA path has no PyTorch fallback)"
            )
        torch.ops.load_library(str(_LIB))
        _loaded = True
    return torch.ops.stb


def check_status(where: str = "") -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait expiry or a bad argument."""
    code = int(load().status_read())
    if code != 0:
        block = load().status_tensor().cpu().tolist()     # {code, peer, expected, observed}
        load().status_reset()
        names = {
            1: "TMA producer gave up waiting for a free pipeline stage",
            2: "MMA issuer gave up waiting for operand tiles",
            3: "epilogue gave up waiting for the accumulator",
            4: "drain wait expired",
            5: "peer flag wait expired (a peer never signalled)",
            6: "attention pipeline wait expired",
            7: "kernel rejected its arguments",
            8: "GEMM gave up waiting for rows of its operand that another CTA was pulling",
        }
        detail = ""
        if code == 5:
            _, peer, expected, observed = block
            detail = f" [group member {peer} silent: waited for epoch {expected}, last saw {observed}]"
        raise RuntimeError(
            f"sm_100a kernel status {code} ({names.get(code, 'unknown')}){detail} {where}")
