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


# kernels launched per op call (ops not listed launch one)
_KERNELS_PER_CALL = {"colsum_bf16": 2, "attention_bwd": 3, "status_read": 0, "status_reset": 0,
                     "layer_forward": 10, "layer_backward": 26, "status_tensor": 0,
                     "layer_forward_sp": 15, "layer_backward_sp": 31,
                     "layer_forward_tp": 12, "layer_backward_tp": 29,
                     "peer_alloc": 0, "peer_free": 0, "device_synchronize": 0, "enable_peer_access": 0, "ipc_handle": 0, "ipc_open": 0,
                     "ipc_close": 0, "tensor_from_ptr": 0}


class CountingOps:
    """Proxy over `torch.ops.stb` that counts this package's kernel launches (benchmarks)."""

    def __init__(self, namespace):
        self._ns = namespace
        self.launches = 0
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            target = getattr(self._ns, name)
            weight = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _t=target, _w=weight):
                self.launches += _w
                return _t(*args)

            self._cache[name] = fn
        return fn


_counter = None


def enable_launch_counting():
    """Make `load()` return a counting proxy (call before the runtime is registered)."""
    global _counter
    if _counter is None:
        _counter = CountingOps(_load_namespace())
    return _counter


def load():
    return _counter if _counter is not None else _load_namespace()


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
