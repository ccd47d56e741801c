"""Profiling target: the fused all-gather GEMMs with a *real* peer on the other end, in ONE process.

    python -m shardtrain_b200.ops.profile_peer_gemm --kind weights --m 512 --n 8960 --k 1536
    python -m shardtrain_b200.ops.profile_peer_gemm --kind sequence --m 1024 --n 4480 --k 1536

The process owns two GPUs.  Half of the operand that the kernel gathers lives on `cuda:1`, the
other half and everything else on `cuda:0`, where the kernel runs; peer access is enabled through
the CUDA runtime, so the kernel's plain loads of the `cuda:1` half cross NVLink.  Nothing waits
on the other GPU (it only holds memory), which makes the process a valid target for a one-kernel
profiler capture: a profiler may replay the launch as often as it likes.  With one visible GPU
both halves are local (`"peer": false` in the output).

Prints one JSON line: CUDA-event time per launch, bytes that crossed the link per launch,
achieved link rate and TFLOP/s, and the relative error against the two-kernel path.
"""

from __future__ import annotations

import argparse
import json

import torch

from shardtrain_b200 import ops as ops_module


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", choices=["weights", "sequence"], default="weights")
    ap.add_argument("--m", type=int, default=512)
    ap.add_argument("--n", type=int, default=8960)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--gated", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    ops = ops_module.load()
    two = torch.cuda.device_count() >= 2 and torch.cuda.can_device_access_peer(0, 1)
    home, away = torch.device("cuda:0"), torch.device("cuda:1" if two else "cuda:0")
    torch.cuda.set_device(home)
    if two:
        torch.zeros(8, device=away)          # creates the context of the second GPU
        ops.enable_peer_access(1)            # kernels on cuda:0 may read cuda:1's memory
        torch.cuda.synchronize()
    gen = torch.Generator(device="cpu").manual_seed(0)
    scrub = torch.empty(64 << 20, dtype=torch.float32, device=home)
    out = {"kind": a.kind, "peer": two, "shape": [a.m, a.n, a.k]}

    if a.kind == "weights":
        rows = a.n // 16 * 16
        W = (torch.randn(rows, a.k, generator=gen) * 0.1).bfloat16()
        if a.gated:
            half = rows // 2
            qh = half * a.k // 2
            parts = [torch.cat([W[:half].reshape(-1)[r * qh:(r + 1) * qh],
                                W[half:].reshape(-1)[r * qh:(r + 1) * qh]]) for r in range(2)]
            table = torch.tensor([[0, qh, half * a.k, 0, 0], [qh, qh, half * a.k, half * a.k, 0]],
                                 dtype=torch.int64)
        else:
            q = rows * a.k // 2
            parts = [W.reshape(-1)[r * q:(r + 1) * q].clone() for r in range(2)]
            table = torch.tensor([[0, q, rows * a.k, 0, 0]], dtype=torch.int64)
        arenas = [parts[0].to(home), parts[1].to(away)]          # rank 1's shard is remote
        ptrs = [t.data_ptr() for t in arenas]
        A = torch.randn(a.m, a.k, generator=gen).bfloat16().to(home)
        full = torch.empty(rows * a.k, device=home, dtype=torch.bfloat16)
        C = torch.empty(a.m, rows, device=home, dtype=torch.bfloat16)
        Hm = torch.empty(a.m, rows // 2, device=home, dtype=torch.bfloat16) if a.gated else None

        def fused():
            ops.gemm_allgather(A, C, None, ptrs, False, table, full, Hm, 0)

        Wd = W.to(home)
        ref = torch.empty_like(C)
        if a.gated:
            ops.gemm_swiglu(A, Wd, ref, torch.empty_like(Hm))
        else:
            ops.gemm(A, Wd, ref, False, False, None, None, False, 1.0, 0)
        link_bytes = rows * a.k * 2 // 2 if two else 0
        flops = 2.0 * a.m * rows * a.k
    else:
        T, seq_local = 2, a.m // 2
        slices = [torch.randn(seq_local, a.k, generator=gen).bfloat16() for _ in range(T)]
        placed = [slices[0].to(home), slices[1].to(away)]
        W = (torch.randn(a.n, a.k, generator=gen) * 0.1).bfloat16().to(home)
        a_dst = torch.empty(a.m, a.k, device=home, dtype=torch.bfloat16)
        C = torch.empty(a.m, a.n, device=home, dtype=torch.bfloat16)

        def fused():
            ops.gemm_seq_pull(a_dst, W, C, False, None, [t.data_ptr() for t in placed], 1, seq_local, 0)

        ref = torch.empty_like(C)
        ops.gemm(torch.cat(slices).to(home), W, ref, False, False, None, None, False, 1.0, 0)
        link_bytes = seq_local * a.k * 2 if two else 0
        flops = 2.0 * a.m * a.n * a.k

    for _ in range(a.warmup):
        fused()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(a.iters):
        scrub.zero_()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fused()
        end.record()
        torch.cuda.synchronize()
        total += begin.elapsed_time(end)
    ms = total / a.iters
    err = ((C.float() - ref.float()).norm() / ref.float().norm()).item()
    ops_module.check_status("profile_peer_gemm")
    out.update(ms=ms, link_bytes=link_bytes, link_gbs=link_bytes / ms / 1e6, tflops=flops / ms / 1e9,
               rel_err_vs_local=err)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
