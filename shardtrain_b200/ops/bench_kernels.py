"""Microbenchmarks of the sm_100a kernels, one kernel family per sub-command.

    python -m shardtrain_b200.ops.bench_kernels gemm --m 4096 --n 17920 --k 1536
    python -m shardtrain_b200.ops.bench_kernels attention --batch 8 --seq 512 --hq 12 --hkv 2
    python -m shardtrain_b200.ops.bench_kernels reduce_scatter_adamw --numel 46797824
    python -m shardtrain_b200.ops.bench_kernels gather_params --numel 46797824

Each prints one JSON line with the CUDA-event time per launch (after warm-up, inputs larger than
the 126 MB L2 or an L2 flush between launches) and the achieved TFLOP/s or GB/s next to the
measured peaks of `MEASURED_PEAKS.json` when that file exists.  `--iters` small (1-3) and
`--warmup 1` make the process suitable as the target of a profiler capture.
"""

from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from shardtrain_b200 import ops as ops_module


def peaks():
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return data.get("hbm_gbs"), data.get("bf16_tflops"), data.get("bf16_tflops_sustained"), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def timed(fn, warmup, iters, flush):
    scrub = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()          # 256 MB written: evicts the 126 MB L2
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += begin.elapsed_time(end)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_swiglu", "gemm_scatter", "gemm_allgather", "gemm_seq_pull",
                                       "attention",
                                       "reduce_scatter_adamw", "gather_params", "gather_shadow",
                                       "rmsnorm"])
    ap.add_argument("--gated", type=int, default=0, help="gemm_allgather: gate|up with SwiGLU epilogue")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=17920)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--a-mn", type=int, default=0)
    ap.add_argument("--b-mn", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--flush", type=int, default=0, help="gemm: scrub the L2 between iterations")
    ap.add_argument("--out-fp32", type=int, default=0, help="gemm: fp32 output (dW / residual stream)")
    ap.add_argument("--staged", type=int, default=1,
                    help="gemm: 1 = outputs leave through staged TMA stores, 0 = per-thread row stores")
    ap.add_argument("--owners", type=int, default=2, help="gemm_scatter: sequence owners (local buffers)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--hq", type=int, default=12)
    ap.add_argument("--hkv", type=int, default=2)
    ap.add_argument("--numel", type=int, default=46797824)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    ops = ops_module.load()
    hbm, burst, sustained, origin = peaks()
    dev = "cuda"
    out = {"kernel": a.kernel, "peaks": origin}
    if a.kernel == "gemm":
        A = torch.randn(a.k if a.a_mn else a.m, a.m if a.a_mn else a.k, device=dev).bfloat16()
        B = torch.randn(a.k if a.b_mn else a.n, a.n if a.b_mn else a.k, device=dev).bfloat16()
        C = torch.empty(a.m, a.n, device=dev, dtype=torch.float32 if a.out_fp32 else torch.bfloat16)
        ms = timed(lambda: ops.gemm(A, B, C, bool(a.a_mn), bool(a.b_mn), None, None, False, 1.0, a.bn,
                                    a.split_k, bool(a.staged)), a.warmup, a.iters, flush=bool(a.flush))
        tflops = 2 * a.m * a.n * a.k / ms / 1e9
        out.update(shape=[a.m, a.n, a.k], a_mn=a.a_mn, b_mn=a.b_mn, out_fp32=a.out_fp32,
                   staged=a.staged, ms=ms, tflops=tflops, output_gbs=C.numel() * C.element_size() / ms / 1e6,
                   frac_of_burst_cublas=tflops / burst, frac_of_sustained_cublas=tflops / sustained)
    elif a.kernel == "gemm_swiglu":
        # gate|up projection: SwiGLU in the GEMM epilogue against GEMM + SwiGLU kernel (--n = 2 x inter)
        inter = a.n // 2
        A = torch.randn(a.m, a.k, device=dev).bfloat16()
        W = (torch.randn(2 * inter, a.k, device=dev) * 0.05).bfloat16()
        C = torch.empty(a.m, 2 * inter, device=dev, dtype=torch.bfloat16)
        Hm = torch.empty(a.m, inter, device=dev, dtype=torch.bfloat16)

        def two():
            ops.gemm(A, W, C, False, False, None, None, False, 1.0, a.bn)
            ops.swiglu_fwd(C, Hm)

        ms_fused = timed(lambda: ops.gemm_swiglu(A, W, C, Hm), a.warmup, a.iters, flush=bool(a.flush))
        ms_two = timed(two, a.warmup, a.iters, flush=bool(a.flush))
        tflops = 2 * a.m * 2 * inter * a.k / ms_fused / 1e9
        out.update(shape=[a.m, 2 * inter, a.k], fused_ms=ms_fused, gemm_then_swiglu_ms=ms_two,
                   tflops=tflops, frac_of_sustained_cublas=tflops / sustained)
    elif a.kernel == "gemm_scatter":
        # row-parallel GEMM with the sequence-scatter epilogue; the owners' receive buffers are
        # local tensors here (the multi-GPU path passes peer pointers to the same kernel)
        A = torch.randn(a.m, a.k, device=dev).bfloat16()
        B = torch.randn(a.k if a.b_mn else a.n, a.n if a.b_mn else a.k, device=dev).bfloat16()
        dest = [torch.empty(a.m // a.owners, a.n, device=dev) for _ in range(a.owners)]
        ptrs = [d.data_ptr() for d in dest]
        ms = timed(lambda: ops.gemm_scatter(A, B, ptrs, a.seq, False, bool(a.b_mn), a.bn), a.warmup,
                   a.iters, flush=False)
        tflops = 2 * a.m * a.n * a.k / ms / 1e9
        out.update(shape=[a.m, a.n, a.k], owners=a.owners, seq=a.seq, ms=ms, tflops=tflops,
                   output_gbs=a.m * a.n * 4 / ms / 1e6, frac_of_sustained_cublas=tflops / sustained)
    elif a.kernel == "gemm_allgather":
        # all-gather fused into the GEMM; the `--owners` ranks' shard arenas are local tensors here
        # (the multi-GPU path hands the same kernel peer pointers), so this measures the kernel's
        # own pipeline without the link.  Compared with gather kernel + GEMM on the same data.
        F = a.owners
        rows = a.n // (8 * F) * (8 * F)
        numel = rows * a.k
        q = numel // F
        W = (torch.randn(rows, a.k, device=dev) * 0.1).bfloat16()
        arenas = [W.reshape(-1)[r * q:(r + 1) * q].clone() for r in range(F)]
        ptrs = [t.data_ptr() for t in arenas]
        A = torch.randn(a.m, a.k, device=dev).bfloat16()
        full = torch.empty(numel, device=dev, dtype=torch.bfloat16)
        side = torch.empty(4, device=dev)
        if a.gated:
            half = rows // 2
            # gate and up are two parameters: each cut into F shards of its own
            qh = half * a.k // F
            arenas = [torch.cat([W[:half].reshape(-1)[r * qh:(r + 1) * qh],
                                 W[half:].reshape(-1)[r * qh:(r + 1) * qh]]) for r in range(F)]
            ptrs = [t.data_ptr() for t in arenas]
            table = torch.tensor([[0, qh, half * a.k, 0, 0], [qh, qh, half * a.k, half * a.k, 0]],
                                 dtype=torch.int64)
            C = torch.empty(a.m, rows, device=dev, dtype=torch.bfloat16)
            Hm = torch.empty(a.m, half, device=dev, dtype=torch.bfloat16)
            fused = lambda: ops.gemm_allgather(A, C, None, ptrs, False, table, full, Hm, 0)   # noqa: E731

            def two():
                ops.gather_params(ptrs, table, full, side, ptrs)
                ops.gemm_swiglu(A, full.view(rows, a.k), C, Hm)
        else:
            table = torch.tensor([[0, q, numel, 0, 0]], dtype=torch.int64)
            C = torch.empty(a.m, rows, device=dev, dtype=torch.bfloat16)
            fused = lambda: ops.gemm_allgather(A, C, None, ptrs, False, table, full, None, a.bn)   # noqa: E731

            def two():
                ops.gather_params(ptrs, table, full, side, ptrs)
                ops.gemm(A, full.view(rows, a.k), C, False, False, None, None, False, 1.0, 0)
        ms_fused = timed(fused, a.warmup, a.iters, flush=True)
        ms_two = timed(two, a.warmup, a.iters, flush=True)
        tflops = 2 * a.m * rows * a.k / ms_fused / 1e9
        out.update(shape=[a.m, rows, a.k], owners=F, gated=a.gated, fused_ms=ms_fused,
                   gather_then_gemm_ms=ms_two, tflops=tflops, weight_gbs=numel * 2 / ms_fused / 1e6,
                   frac_of_sustained_cublas=tflops / sustained)
    elif a.kernel == "gemm_seq_pull":
        # sequence all-gather fused into the GEMM: `--owners` local slices stand in for the peers'
        T = a.owners
        sl = a.m // T
        slices = [torch.randn(sl, a.k, device=dev).bfloat16() for _ in range(T)]
        ptrs = [t.data_ptr() for t in slices]
        B = (torch.randn(a.n, a.k, device=dev) * 0.1).bfloat16()
        A_dst = torch.empty(T * sl, a.k, device=dev, dtype=torch.bfloat16)
        C = torch.empty(T * sl, a.n, device=dev, dtype=torch.bfloat16)
        ms_fused = timed(lambda: ops.gemm_seq_pull(A_dst, B, C, False, None, ptrs, 1, sl, a.bn),
                         a.warmup, a.iters, flush=True)

        def two():
            ops.seq_gather(ptrs, A_dst, 1, sl, a.k * 2)
            ops.gemm(A_dst, B, C, False, False, None, None, False, 1.0, a.bn)
        ms_two = timed(two, a.warmup, a.iters, flush=True)
        ms_gemm = timed(lambda: ops.gemm(A_dst, B, C, False, False, None, None, False, 1.0, a.bn),
                        a.warmup, a.iters, flush=True)
        tflops = 2 * T * sl * a.n * a.k / ms_fused / 1e9
        out.update(shape=[T * sl, a.n, a.k], owners=T, fused_ms=ms_fused, gather_then_gemm_ms=ms_two,
                   gemm_only_ms=ms_gemm, tflops=tflops, frac_of_sustained_cublas=tflops / sustained)
    elif a.kernel == "attention":
        D, W = 128, (a.hq + 2 * a.hkv) * 128
        rows = a.batch * a.seq
        qkv = (torch.randn(rows, W, device=dev) * 0.5).bfloat16()
        o = torch.empty(rows, a.hq * D, device=dev, dtype=torch.bfloat16)
        do = torch.randn_like(o)
        lse = torch.empty(a.batch, a.hq, a.seq, device=dev)
        delta, dqkv = torch.empty_like(lse), torch.empty_like(qkv)
        # scratch for the dK/dV head-group split (same sizing as the layer executor)
        scratch = torch.empty((a.hq // a.hkv) * rows * 2 * a.hkv * D, device=dev)
        scale = 1 / math.sqrt(D)
        fwd = timed(lambda: ops.attention_fwd(qkv, o, lse, None, a.batch, a.seq, a.hq, a.hkv, scale),
                    a.warmup, a.iters, flush=True)
        bwd = timed(lambda: ops.attention_bwd(qkv, o, do, lse, delta, dqkv, scratch, None, a.batch, a.seq,
                                              a.hq, a.hkv, scale), a.warmup, a.iters, flush=True)
        flops = 4 * a.batch * a.hq * a.seq * a.seq * D / 2      # causal: half the score matrix
        out.update(batch=a.batch, seq=a.seq, hq=a.hq, hkv=a.hkv, fwd_ms=fwd, bwd_ms=bwd,
                   fwd_tflops=flops / fwd / 1e9, bwd_tflops=2.5 * flops / bwd / 1e9,
                   fwd_frac_of_burst_cublas=flops / fwd / 1e9 / burst)
    elif a.kernel == "gather_shadow":
        n = a.numel // 8 * 8
        table = torch.tensor([[0, n, n, 0, 0]], dtype=torch.int64)
        shard = torch.randn(n, device=dev)
        shadow = shard.bfloat16()
        fb, ff = torch.empty(n, device=dev, dtype=torch.bfloat16), torch.empty(4, device=dev)
        ms = timed(lambda: ops.gather_params([shard.data_ptr()], table, fb, ff, [shadow.data_ptr()]),
                   a.warmup, a.iters, True)
        moved = n * (2 + 2)
        out.update(numel=n, ms=ms, gbs=moved / ms / 1e6, frac_of_copy_peak=moved / ms / 1e6 / hbm)
    elif a.kernel in ("reduce_scatter_adamw", "gather_params"):
        n = a.numel // 4 * 4
        table = torch.tensor([[0, n, n, 0, 0]], dtype=torch.int64)
        if a.kernel == "gather_params":
            shard = torch.randn(n, device=dev)
            fb, ff = torch.empty(n, device=dev, dtype=torch.bfloat16), torch.empty(4, device=dev)
            ms = timed(lambda: ops.gather_params([shard.data_ptr()], table, fb, ff), a.warmup, a.iters, True)
            moved = n * (4 + 2)
        else:
            full = torch.randn(n, device=dev)
            g, p = torch.zeros(n, device=dev), torch.randn(n, device=dev)
            m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            flags = torch.zeros(2, device=dev, dtype=torch.int32)
            ms = timed(lambda: ops.reduce_scatter_adamw([full.data_ptr()], 0, table, g, p, m, v, 1.0, True,
                                                        1e-5, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, flags),
                       a.warmup, a.iters, True)
            moved = n * 4 * (1 + 2 + 6)     # slot read; grad read+write; p, m, v read+write
        out.update(numel=n, ms=ms, gbs=moved / ms / 1e6, frac_of_copy_peak=moved / ms / 1e6 / hbm)
    else:
        rows, cols = a.m, a.k
        x, w = torch.randn(rows, cols, device=dev), torch.randn(cols, device=dev)
        y, inv = torch.empty(rows, cols, device=dev, dtype=torch.bfloat16), torch.empty(rows, device=dev)
        ms = timed(lambda: ops.rmsnorm_fwd(x, w, y, inv, 1e-6), a.warmup, a.iters, True)
        moved = rows * cols * 6
        out.update(rows=rows, cols=cols, ms=ms, gbs=moved / ms / 1e6, frac_of_copy_peak=moved / ms / 1e6 / hbm)
    torch.cuda.synchronize()
    ops_module.check_status("bench_kernels")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
