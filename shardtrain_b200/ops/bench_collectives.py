"""Fused compute+collective kernels against the NCCL(+cuBLAS) path, in one process group.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m shardtrain_b200.ops.bench_collectives [--quick] [--only fa,fb,fc,fd]

Four sweeps, each row timed both ways on the same buffers:

* `fa`  parameter all-gather -> GEMM (M = 512 activation rows, K = 1536): unit sizes 1 MB - 1 GB
        of FP32 parameters.  ours: `gemm_allgather` (weights pulled inside the GEMM), and the
        two-kernel form `gather_params` + `gemm`; NCCL: `all_gather_into_tensor` (FP32) + cast +
        `torch.matmul`.
* `fb`  gradient reduce-scatter -> FP32 accumulate -> AdamW: unit sizes 1 MB - 1 GB.  ours: flag
        barrier + `reduce_scatter_adamw`; NCCL: `reduce_scatter_tensor` + fused torch AdamW on
        the shard.
* `fc`  sequence all-gather -> column GEMM and `fd` row GEMM -> sequence reduce-scatter, with
        M in {512, 2048, 8192}, K in {1536, 3584}, N in {1536, 8960, 18944}.  ours: `seq_gather` +
        `gemm` / `gemm_scatter` + barrier + `slot_sum_rmsnorm`; NCCL: `all_gather_into_tensor` /
        `reduce_scatter_tensor` around `torch.matmul`.

Every time is CUDA-event time on the launching stream after warm-up, maximum over ranks, with a
256 MB scrub of the L2 between iterations.  `floor_us` is the roofline of the row: the slower of
FLOPs at the measured cuBLAS bf16 peak and bytes that must enter this GPU over NVLink at the
measured peer-copy rate (770 GB/s per direction); `frac` = floor / measured.  Rank 0 prints one
JSON line per row and, with `--table PATH`, writes a markdown table.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from shardtrain_b200 import ops as ops_module
from shardtrain_b200.distributed.peer import PeerMemory

NVLINK_GBS = 770.0       # measured peer copy per direction on this pool (nominal 900)
MB = 1 << 20


def peaks():
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class Timer:
    def __init__(self, device, warmup, iters):
        self.device, self.warmup, self.iters = device, warmup, iters
        self.scrub = torch.empty(64 * MB, dtype=torch.float32, device=device)

    def __call__(self, fn) -> float:
        """Mean microseconds per call, maximum over ranks."""
        for _ in range(self.warmup):
            fn()
        total = 0.0
        for _ in range(self.iters):
            self.scrub.zero_()
            if dist.get_world_size() > 1:
                dist.barrier()
            torch.cuda.synchronize(self.device)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            fn()
            end.record()
            torch.cuda.synchronize(self.device)
            total += begin.elapsed_time(end)
        mean = torch.tensor([total / self.iters * 1e3], device=self.device, dtype=torch.float64)
        if dist.get_world_size() > 1:
            dist.all_reduce(mean, op=dist.ReduceOp.MAX)
        return float(mean.item())


def floor_us(flops, link_bytes, tflops):
    return max(flops / (tflops * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e6


def sweep_fa(ops, peer, timer, sizes_mb, tflops, emit):
    """Parameter all-gather fused into the consuming GEMM."""
    F, rank, dev = peer.degree, peer.rank, peer.device
    M, K = 512, 1536
    for size_mb in sizes_mb:
        rows = max(F * 8, (size_mb * MB // 4) // K // (F * 8) * (F * 8))   # shards end on row groups
        numel = rows * K
        q = numel // F
        shard_buf = peer.alloc(q * 4)            # fp32 master shard (for the NCCL arm)
        shadow_buf = peer.alloc(q * 2)           # bf16 shadow of it (what our kernels pull)
        shard = shard_buf.tensor(ops, q) if F > 1 else shard_buf.owner.view(torch.float32)[:q]
        shadow = (shadow_buf.tensor(ops, q, torch.bfloat16) if F > 1
                  else shadow_buf.owner.view(torch.bfloat16)[:q])
        shard.normal_(generator=torch.Generator(device=dev).manual_seed(rank)).mul_(0.05)
        shadow.copy_(shard)
        torch.cuda.synchronize(dev)
        if F > 1:
            dist.barrier()
        table = torch.tensor([[0, q, numel, 0, 0]], dtype=torch.int64)
        a = torch.randn(M, K, device=dev).bfloat16()
        full = torch.empty(numel, device=dev, dtype=torch.bfloat16)
        side = torch.empty(4, device=dev)
        out = torch.empty(M, rows, device=dev, dtype=torch.bfloat16)

        def fused():
            ops.gemm_allgather(a, out, None, shadow_buf.ptrs, False, table, full, None, 0)

        def two_kernels():
            ops.gather_params(shard_buf.ptrs, table, full, side, shadow_buf.ptrs)
            ops.gemm(a, full.view(rows, K), out, False, False, None, None, False, 1.0, 0)

        gathered = torch.empty(numel, device=dev)

        def nccl():
            if F > 1:
                dist.all_gather_into_tensor(gathered, shard)
            else:
                gathered.copy_(shard)
            torch.matmul(a, gathered.view(rows, K).to(torch.bfloat16).t(), out=out)

        t_fused, t_two, t_nccl = timer(fused), timer(two_kernels), timer(nccl)
        reference = out.clone()
        fused()
        torch.cuda.synchronize(dev)
        err = ((out.float() - reference.float()).norm() / reference.float().norm()).item()
        flops = 2.0 * M * rows * K
        link = numel * 2 * (F - 1) / F            # bf16 bytes that enter this GPU
        floor = floor_us(flops, link, tflops)
        emit(dict(sweep="fa_allgather_gemm", unit_mb_fp32=size_mb, M=M, N=rows, K=K, ranks=F,
                  fused_us=t_fused, gather_then_gemm_us=t_two, nccl_cublas_us=t_nccl,
                  floor_us=floor, frac=floor / t_fused, vs_nccl=t_nccl / t_fused,
                  link_gbs=link / t_fused / 1e3, rel_err_vs_nccl=err))
        del shard, shadow


def sweep_fb(ops, peer, timer, sizes_mb, tflops, emit, nvls=False):
    """Gradient reduce-scatter fused with accumulate + AdamW."""
    F, rank, dev = peer.degree, peer.rank, peer.device
    for size_mb in sizes_mb:
        numel = max(F * 4, (size_mb * MB // 4) // (F * 4) * (F * 4))
        q = numel // F
        slot = peer.alloc_multicast(numel * 4) if nvls else peer.alloc(numel * 4)
        grads = slot.tensor(ops, numel) if F > 1 else slot.owner.view(torch.float32)[:numel]
        grads.normal_()
        table = torch.tensor([[0, q, numel, 0, 0]], dtype=torch.int64)
        g, p = torch.zeros(q, device=dev), torch.randn(q, device=dev)
        m, v = torch.zeros(q, device=dev), torch.zeros(q, device=dev)
        shadow = torch.empty(q, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(2, device=dev, dtype=torch.int32)
        torch.cuda.synchronize(dev)

        def ours(multicast=0):
            peer.barrier("fsdp_rs")
            ops.reduce_scatter_adamw(slot.ptrs, rank, table, g, p, m, v, 1.0 / F, False, 1e-5, 0.9,
                                     0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, flags, 1, 0, 1.0, shadow,
                                     multicast)

        leaf = torch.nn.Parameter(torch.randn(q, device=dev))
        leaf.grad = torch.zeros(q, device=dev)
        opt = torch.optim.AdamW([leaf], lr=1e-5, fused=True)
        reduced = torch.empty(q, device=dev)

        def nccl():
            if F > 1:
                dist.reduce_scatter_tensor(reduced, grads)
            else:
                reduced.copy_(grads)
            leaf.grad.copy_(reduced.div_(F))
            opt.step()

        t_ours, t_nccl = timer(ours), timer(nccl)
        t_nvls = None
        if slot.multicast_ptr:
            # same reduction through the switch; the two must agree to fp32 summation order
            p_ref = p.clone()
            ours()
            after_p2p = g.clone()
            p.copy_(p_ref)
            ours(slot.multicast_ptr)
            torch.cuda.synchronize(dev)
            nvls_err = ((g - after_p2p).abs().max() / after_p2p.abs().max().clamp_min(1e-12)).item()
            t_nvls = timer(lambda: ours(slot.multicast_ptr))
        link = q * 4 * (F - 1)                    # this rank's slice pulled from every peer
        hbm = q * 4 * (F + 8) + q * 2             # slots read; g, p, m, v read + written; shadow
        floor = max(link / (NVLINK_GBS * 1e9), hbm / 6.5e12) * 1e6
        emit(dict(sweep="fb_reduce_scatter_adamw", unit_mb_fp32=size_mb, numel=numel, ranks=F,
                  fused_us=t_ours, nccl_adamw_us=t_nccl, floor_us=floor, frac=floor / t_ours,
                  vs_nccl=t_nccl / t_ours, link_gbs=link / t_ours / 1e3,
                  fused_nvls_us=t_nvls if t_nvls is not None else "n/a",
                  nvls_vs_p2p_max_rel_diff=nvls_err if t_nvls is not None else "n/a"))
        del grads


def sweep_fc_fd(ops, peer, timer, shapes, tflops, emit, which):
    """Sequence-parallel all-gather -> GEMM (fc) and GEMM -> reduce-scatter (fd)."""
    T, rank, dev = peer.degree, peer.rank, peer.device
    for M, K, N in shapes:
        seq, batch = 512, M // 512
        sl = seq // T
        rows_local = batch * sl
        if "fc" in which:
            act = peer.alloc(rows_local * K * 2)
            x = (act.tensor(ops, rows_local * K, torch.bfloat16) if T > 1
                 else act.owner.view(torch.bfloat16)[:rows_local * K]).view(rows_local, K)
            x.normal_()
            w = torch.randn(N // T, K, device=dev).bfloat16()       # column-parallel slice
            full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M, N // T, device=dev, dtype=torch.bfloat16)
            torch.cuda.synchronize(dev)

            def ours():
                peer.barrier("sp_ag")
                ops.seq_gather(act.ptrs, full, batch, sl, K * 2)
                ops.gemm(full, w, out, False, False, None, None, False, 1.0, 0)

            packed = torch.empty(T * rows_local, K, device=dev, dtype=torch.bfloat16)

            def nccl():
                if T > 1:
                    dist.all_gather_into_tensor(packed.view(-1), x.reshape(-1))
                    gathered = packed.view(T, batch, sl, K).movedim(0, 1).reshape(M, K)
                else:
                    gathered = x
                torch.matmul(gathered, w.t(), out=out)

            t_ours, t_nccl = timer(ours), timer(nccl)
            flops = 2.0 * M * (N // T) * K
            link = rows_local * K * 2 * (T - 1)
            floor = floor_us(flops, link, tflops)
            emit(dict(sweep="fc_seq_allgather_gemm", M=M, K=K, N=N, ranks=T, ours_us=t_ours,
                      nccl_cublas_us=t_nccl, floor_us=floor, frac=floor / t_ours,
                      vs_nccl=t_nccl / t_ours))
        if "fd" in which and T > 1:
            a = torch.randn(M, K // T, device=dev).bfloat16()        # row-parallel input slice
            w = torch.randn(N, K // T, device=dev).bfloat16()
            recv = peer.alloc(T * rows_local * N * 4)
            slots = recv.tensor(ops, T * rows_local * N).view(T, rows_local, N)
            push = [p + rank * rows_local * N * 4 for p in recv.ptrs]
            summed = torch.empty(rows_local, N, device=dev)
            torch.cuda.synchronize(dev)

            def ours():
                ops.gemm_scatter(a, w, push, seq, False, False, 0)
                peer.barrier("sp_rs")
                ops.slot_sum_rmsnorm(slots, None, summed, None, None, None, 0.0)
                peer.barrier("sp_rs")      # slots may be overwritten only after every reader

            partial = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            reduced = torch.empty(sl, batch, N, device=dev, dtype=torch.bfloat16)

            def nccl():
                torch.matmul(a, w.t(), out=partial)
                packed = partial.view(batch, seq, N).movedim(1, 0).contiguous()
                dist.reduce_scatter_tensor(reduced.view(-1), packed.view(-1))

            t_ours, t_nccl = timer(ours), timer(nccl)
            flops = 2.0 * M * N * (K // T)
            link = rows_local * N * 4 * (T - 1)                      # fp32 partial rows received
            floor = floor_us(flops, link, tflops)
            emit(dict(sweep="fd_gemm_seq_reduce_scatter", M=M, K=K, N=N, ranks=T, ours_us=t_ours,
                      nccl_cublas_us=t_nccl, floor_us=floor, frac=floor / t_ours,
                      vs_nccl=t_nccl / t_ours, note="ours reduces fp32 partial sums, NCCL arm bf16"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="three sizes / four shapes per sweep")
    ap.add_argument("--only", default="fa,fb,fc,fd")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--table", default="")
    ap.add_argument("--nvls", action="store_true",
                    help="fb: also time the reduction through the NVSwitch (multicast-bound slots)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    ops = ops_module.load()
    peer = PeerMemory(dist.group.WORLD if world > 1 else None, device, ops, wait_seconds=5.0)
    timer = Timer(device, a.warmup, a.iters)
    tflops, origin = peaks()
    rows = []

    def emit(row):
        row["peaks"] = origin
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    which = set(a.only.split(","))
    sizes = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024]
    shapes = [(m, k, n) for m in (512, 2048, 8192) for k in (1536, 3584) for n in (1536, 8960, 18944)]
    if a.quick:
        sizes = [1, 32, 256]
        shapes = [(512, 1536, 8960), (2048, 1536, 8960), (8192, 3584, 18944), (512, 3584, 1536)]
    sizes = [s for s in sizes if s <= a.max_mb]
    try:
        if "fa" in which:
            sweep_fa(ops, peer, timer, sizes, tflops, emit)
        if "fb" in which:
            sweep_fb(ops, peer, timer, sizes, tflops, emit, nvls=a.nvls)
        if which & {"fc", "fd"}:
            sweep_fc_fd(ops, peer, timer, shapes, tflops, emit, which)
        torch.cuda.synchronize(device)
        ops_module.check_status("bench_collectives")
        if rank == 0 and a.table:
            write_table(Path(a.table), rows, world)
    finally:
        if world > 1:
            dist.barrier()
        peer.close()
        dist.destroy_process_group()


def write_table(path: Path, rows, world):
    lines = [f"# Fused collectives vs NCCL(+cuBLAS), {world} GPUs", "",
             "Times in microseconds (CUDA events, max over ranks, L2 scrubbed between iterations); "
             "`frac` = roofline floor / measured, floor = max(FLOPs at the measured cuBLAS bf16 "
             f"peak, NVLink bytes in at {NVLINK_GBS:.0f} GB/s).", ""]
    by_sweep: dict[str, list] = {}
    for row in rows:
        by_sweep.setdefault(row["sweep"], []).append(row)
    for sweep, members in by_sweep.items():
        keys = [k for k in members[0] if k not in ("sweep", "peaks", "note")]
        lines += [f"## {sweep}", "", "| " + " | ".join(keys) + " |", "|" + "---|" * len(keys)]
        for row in members:
            cells = [f"{row[k]:.3g}" if isinstance(row[k], float) else str(row[k]) for k in keys]
            lines.append("| " + " | ".join(cells) + " |")
        lines.append("")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text("\n".join(lines))


if __name__ == "__main__":
    main()
