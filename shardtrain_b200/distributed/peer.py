"""NVLink peer memory for one process group: CUDA IPC allocations every member can address,
and a flag-based barrier kernel that orders kernels across GPUs.

`PeerMemory.alloc(nbytes)` cudaMallocs a zeroed buffer, exchanges its IPC handle inside the group
(`all_gather_object` over the group's own communicator) and returns a `PeerBuffer` with the local
pointer and one device pointer per member (this rank's entry is the local pointer).  The fused
kernels take those pointer tables; through NVSwitch every peer is one hop away at full bandwidth.

`barrier(channel)` launches a 1-CTA kernel on the current stream: it publishes a new epoch to
every peer's flag pad (`st.release.sys`) and waits until every peer has published the same epoch
to this rank's pad.  The wait is bounded in *time* (`wait_seconds`, seconds rather than minutes;
derived from `debug.distributed_timeout_seconds` by the executor): when it runs out the kernel
records a status block and returns, `ops.check_status()` raises on the host, and every barrier
already queued behind it returns at once instead of spinning its own budget.  Each logical
channel has its own flag slot and its own epoch counter; all members must call the barriers of a
channel in the same order.  With one member every call is a no-op and buffers are ordinary
device tensors.

Teardown: an exported buffer is freed only after every member has said (on the host, through the
group's store-backed `all_gather_object`, which the group's timeout bounds) that its device is
idle and its imports are closed.  When that handshake cannot complete -- a member failed, the
caller says the run failed -- nothing is freed: the buffers stay mapped until the process exits,
so a peer kernel that is still reading them never sees freed memory.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

CHANNEL_SLOTS = {"fsdp_ag": 0, "fsdp_rs": 1, "sp_ag": 2, "sp_rs": 3, "step": 4, "misc": 5,
                 "metrics": 6}
METRIC_WIDTH = 16            # doubles per small all-reduce (csrc/peer.cu: kMetricWidth)
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2, torch.uint8: 3}


@dataclass
class PeerBuffer:
    local_ptr: int
    ptrs: list[int]          # one device pointer per group member, index = group rank
    nbytes: int
    owner: object = None     # keeps an ordinary tensor alive in the single-member case
    multicast_ptr: int = 0   # NVLS: one address that reaches every member's copy (0 = none)

    def tensor(self, ops, numel: int, dtype=torch.float32, offset_bytes: int = 0) -> torch.Tensor:
        return ops.tensor_from_ptr(self.local_ptr + offset_bytes, numel, _DTYPE_CODE[dtype])


class PeerMemory:
    MAX_WAIT_SECONDS = 10.0     # upper clamp of any device-side wait

    def __init__(self, group, device, ops, *, wait_seconds: float = 2.0):
        self.group, self.device, self.ops = group, torch.device(device), ops
        live = dist.is_initialized() and group is not None
        self.degree = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        if wait_seconds <= 0:
            raise ValueError("wait_seconds must be positive")
        # microseconds handed to the kernels; seconds, never minutes, on a shared GPU
        self.wait_us = max(1, int(min(wait_seconds, self.MAX_WAIT_SECONDS) * 1e6))
        self.closed = False
        self.epochs = {name: 0 for name in CHANNEL_SLOTS}
        self._allocations: list[PeerBuffer] = []
        self._opened: list[int] = []
        self._multicast: list[PeerBuffer] = []    # kept until process exit (see alloc_multicast)
        self.multicast_refusal = None
        self.flags = self.alloc(4096) if self.degree > 1 else None
        # inbox of the small all-reduce: [2 parities][8 senders][METRIC_WIDTH] doubles
        self.inbox = self.alloc(2 * 8 * METRIC_WIDTH * 8) if self.degree > 1 else None

    def alloc(self, nbytes: int) -> PeerBuffer:
        nbytes = -(-int(nbytes) // 512) * 512
        if self.degree == 1:
            owner = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            buf = PeerBuffer(owner.data_ptr(), [owner.data_ptr()], nbytes, owner)
            self._allocations.append(buf)
            return buf
        local = int(self.ops.peer_alloc(nbytes))
        handle = self.ops.ipc_handle(local)
        gathered: list = [None] * self.degree
        dist.all_gather_object(gathered, bytes(handle.numpy().tobytes()), group=self.group)
        ptrs = []
        for member, raw in enumerate(gathered):
            if member == self.rank:
                ptrs.append(local)
            else:
                opened = int(self.ops.ipc_open(torch.frombuffer(bytearray(raw), dtype=torch.uint8)))
                self._opened.append(opened)
                ptrs.append(opened)
        buf = PeerBuffer(local, ptrs, nbytes)
        self._allocations.append(buf)
        return buf

    def alloc_multicast(self, nbytes: int) -> PeerBuffer:
        """Like `alloc`, for buffers that kernels also address through NVLS (`multimem.*`): the
        memory comes from torch's symmetric-memory allocator, which binds it to an NVLink
        multicast object spanning the group when the driver and the fabric allow it.  When they
        do not (no NVSwitch, multicast refused, symmetric memory unavailable) this silently
        returns an ordinary peer buffer with `multicast_ptr == 0`, and callers keep to plain
        peer loads.  The tensor is never returned to torch before process exit."""
        if self.degree == 1:
            return self.alloc(nbytes)
        nbytes = -(-int(nbytes) // 512) * 512
        try:
            import torch.distributed._symmetric_memory as symm_mem

            tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            handle = symm_mem.rendezvous(tensor, self.group)
            multicast = int(handle.multicast_ptr)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            if not multicast or len(ptrs) != self.degree:
                raise RuntimeError("no multicast address")
        except Exception as exc:  # noqa: BLE001 - any refusal means: plain peer memory
            self.multicast_refusal = f"{type(exc).__name__}: {exc}"
            # every member must take the same branch: agree on the outcome
            verdicts: list = [None] * self.degree
            dist.all_gather_object(verdicts, False, group=self.group)
            return self.alloc(nbytes)
        verdicts = [None] * self.degree
        dist.all_gather_object(verdicts, True, group=self.group)
        if not all(verdicts):
            return self.alloc(nbytes)
        tensor.zero_()
        buf = PeerBuffer(ptrs[self.rank], ptrs, nbytes, owner=(tensor, handle),
                         multicast_ptr=multicast)
        self._multicast.append(buf)
        return buf

    def barrier(self, channel: str) -> None:
        """Enqueue a cross-GPU barrier on the current stream (no-op for a single member)."""
        if self.degree == 1:
            return
        self.epochs[channel] += 1
        self.ops.peer_barrier(self.flags.ptrs, self.rank, self.epochs[channel],
                              CHANNEL_SLOTS[channel], self.wait_us)

    def all_reduce_small(self, values: torch.Tensor, min_mask: int = 0) -> torch.Tensor:
        """SUM (or MIN where bit i of `min_mask` is set) of a float64 vector of at most
        METRIC_WIDTH elements over the group, in one kernel on the current stream; every member
        gets bit-identical results.  Members must call in the same order."""
        if values.dtype != torch.float64 or values.numel() > METRIC_WIDTH:
            raise ValueError("all_reduce_small takes at most 16 float64 values")
        if self.degree == 1:
            return values.clone()
        out = torch.empty_like(values)
        self.epochs["metrics"] += 1
        self.ops.peer_allreduce_small(self.flags.ptrs, self.inbox.ptrs, self.rank,
                                      self.epochs["metrics"], CHANNEL_SLOTS["metrics"],
                                      values.contiguous(), out, min_mask, self.wait_us)
        return out

    def close(self, *, failed: bool = False) -> bool:
        """Release the peer mappings.  Returns True when the exported buffers were freed.

        Order: (1) this rank's device goes idle, (2) its imports of the peers' buffers are
        closed, (3) every member reports both on the host, (4) only then are the exported
        buffers freed.  With `failed=True`, or when step 3 raises (a member is gone, the group's
        timeout ran out), steps 2-4 are skipped for the exported buffers: they are leaked until
        the process exits, because a peer may still have a kernel in flight that reads them.
        """
        if self.closed:
            return False
        self.closed = True
        if self.degree == 1:
            self._allocations.clear()
            return True
        if failed:
            self._leak()
            return False
        try:
            self.ops.device_synchronize()
            for ptr in self._opened:
                self.ops.ipc_close(ptr)
            self._opened.clear()
            reports: list = [None] * self.degree
            dist.all_gather_object(reports, ("idle", self.rank), group=self.group)
            if any(r is None or r[0] != "idle" for r in reports):
                raise RuntimeError("a member did not report an idle device")
        except Exception:  # noqa: BLE001 - any failure of the handshake means: do not free
            self._leak()
            return False
        for buf in self._allocations:
            if buf.owner is None:
                self.ops.peer_free(buf.local_ptr)
        self._allocations.clear()
        return True

    def _leak(self) -> None:
        """Forget the bookkeeping without freeing: the driver reclaims at process exit."""
        self._opened.clear()
        self._allocations.clear()
