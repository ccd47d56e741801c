"""sm_100a kernels against plain PyTorch FP32 references of the same op (run with -m gpu)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from shardtrain_b200 import ops as module

    namespace = module.load()      # raises if the in-tree extension is missing: no fallback
    yield namespace
    torch.cuda.synchronize()
    module.check_status("kernel tests")


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def close_on_edges(got, want, *, atol, rtol, width=9):
    """Elementwise comparison of the first / last rows and columns of a matrix: a norm ratio does
    not notice a few wrong elements at a ragged tile edge."""
    got, want = got.float(), want.float()
    for part in (slice(0, width), slice(-width, None)):
        torch.testing.assert_close(got[part], want[part], atol=atol, rtol=rtol)
        torch.testing.assert_close(got[:, part], want[:, part], atol=atol, rtol=rtol)


GEMM_CASES = [
    # M, N, K, a_mn, b_mn, out_fp32, bias, residual, accumulate, force_bn
    (128, 128, 64, False, False, False, False, False, False, 128),
    (256, 256, 512, False, False, False, False, False, False, 256),
    (512, 2048, 1536, False, False, False, True, False, False, 0),
    (512, 1536, 8960, False, False, True, False, True, False, 0),
    (200, 328, 192, False, False, False, True, True, False, 0),
    (512, 1536, 2048, False, True, True, False, False, False, 0),
    (256, 256, 128, False, True, False, False, False, False, 128),
    (2048, 1536, 512, True, True, True, False, False, True, 0),
    (1000, 520, 264, True, True, True, False, False, False, 256),
    (4096, 1536, 8960, False, False, False, False, False, False, 256),   # several tiles per CTA
    (4096, 1536, 2048, False, False, True, False, True, False, 192),     # 192-wide tiles, 2 waves
    (2048, 1536, 2048, False, True, True, False, False, False, 0),       # heuristic picks 192
    (2048, 1536, 1024, True, True, True, False, False, False, 192),
    (300, 584, 328, False, False, False, True, True, False, 192),        # ragged edges
]


@pytest.mark.parametrize("case", GEMM_CASES, ids=[f"{c[0]}x{c[1]}x{c[2]}_{int(c[3])}{int(c[4])}" for c in GEMM_CASES])
def test_tcgen05_gemm(ops, case):
    M, N, K, a_mn, b_mn, out_fp32, bias, resid, acc, bn = case
    torch.manual_seed(0)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    out = torch.zeros(M, N, device=DEV, dtype=torch.float32 if out_fp32 else torch.bfloat16)
    bias_t = torch.randn(N, device=DEV) if bias else None
    res_t = torch.randn(M, N, device=DEV).to(out.dtype) if resid else None
    if acc:
        out.normal_()
        ref = ref + out.float()
    if bias:
        ref = ref + bias_t
    if resid:
        ref = ref + res_t.float()
    ops.gemm(a, b, out, a_mn, b_mn, bias_t, res_t, acc, 1.0, bn)
    assert rel(out, ref) < (2e-5 if out_fp32 else 4e-3)
    # bf16 operands are exact in fp32, products accumulate in fp32: only the output rounding and
    # the summation order separate the kernel from the reference
    scale = math.sqrt(K)
    close_on_edges(out, ref, atol=(2e-4 if out_fp32 else 2e-2) * scale, rtol=1e-5 if out_fp32 else 1e-2)


@pytest.mark.parametrize("out_fp32", [False, True], ids=["bf16", "fp32"])
@pytest.mark.parametrize("shape", [(300, 584, 328, 192), (512, 17920, 512, 256), (130, 40, 64, 128),
                                   (1000, 520, 264, 0)], ids=lambda s: "x".join(map(str, s)))
def test_gemm_staged_tma_store_equals_row_stores_and_stays_inside_the_output(ops, shape, out_fp32):
    """Plain outputs leave through TMA stores of 32-row boxes staged in shared memory.  Same bits
    as the per-thread row stores; a box that overhangs the ragged edge of the output (rows past
    M, columns past N) must not touch the memory around it."""
    M, N, K, bn = shape
    torch.manual_seed(3)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    dtype = torch.float32 if out_fp32 else torch.bfloat16
    bias = torch.randn(N, device=DEV)
    pitch = N + 24                                    # columns N.. of every row are a guard band
    res = torch.randn(M, pitch, device=DEV).to(dtype)[:, :N]      # same row pitch as the output
    outs = []
    for staged in (False, True):
        plane = torch.full((M + 40, pitch), 7.0, device=DEV, dtype=dtype)
        out = plane[:M, :N]
        ops.gemm(a, b, out, False, False, bias, res, False, 1.0, bn, 1, staged)
        assert torch.all(plane[M:] == 7.0) and torch.all(plane[:, N:] == 7.0)
        outs.append(out.clone())
    assert torch.equal(outs[0], outs[1])
    want = a.float() @ b.float().t() + bias + res.float()
    close_on_edges(outs[1], want, atol=(2e-4 if out_fp32 else 2e-2) * math.sqrt(K),
                   rtol=1e-5 if out_fp32 else 1e-2)


SPLIT_CASES = [
    # M, N, K, a_mn, b_mn, out_fp32, bias, residual, force_bn, split_k
    (512, 1536, 8960, False, False, True, False, True, 256, 0),     # 24 tiles -> 6-way split
    (4096, 1536, 4096, False, True, True, False, False, 256, 0),    # 148 whole + 44 tiles x 3
    (640, 520, 1104, False, False, False, True, True, 128, 4),      # ragged, bf16 out, bias
    (1024, 1536, 2048, True, True, True, False, False, 0, 0),
]


@pytest.mark.parametrize("case", SPLIT_CASES, ids=[f"{c[0]}x{c[1]}x{c[2]}_s{c[9]}" for c in SPLIT_CASES])
def test_gemm_tail_split_is_deterministic_and_matches_unsplit(ops, case):
    """Tail tiles cut along K, reduced by the last arriving CTA in split order: equal (to fp32
    rounding) to the unsplit kernel, bit-identical run to run, and the counters reset themselves."""
    M, N, K, a_mn, b_mn, out_fp32, bias, residual, bn, split = case
    torch.manual_seed(1)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV).bfloat16()
    dtype = torch.float32 if out_fp32 else torch.bfloat16
    bias_t = torch.randn(N, device=DEV) if bias else None
    res = torch.randn(M, N, device=DEV).to(dtype) if residual else None
    outs = []
    for split_k in (1, split, split):
        out = torch.empty(M, N, device=DEV, dtype=dtype)
        ops.gemm(a, b, out, a_mn, b_mn, bias_t, res, False, 1.0, bn, split_k)
        outs.append(out)
    assert torch.equal(outs[1], outs[2])
    assert rel(outs[1], outs[0]) < (1e-5 if out_fp32 else 4e-3)
    want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    want = want + (bias_t if bias else 0) + (res.float() if residual else 0)
    assert rel(outs[1], want) < 5e-3
    close_on_edges(outs[1], want, atol=(2e-4 if out_fp32 else 2e-2) * math.sqrt(K),
                   rtol=1e-5 if out_fp32 else 1e-2)


def test_gemm_rejects_bad_arguments(ops):
    a = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.gemm(a, torch.zeros(128, 72, device=DEV, dtype=torch.bfloat16),
                 torch.zeros(128, 128, device=DEV, dtype=torch.bfloat16), False, False, None, None,
                 False, 1.0, 0)
    with pytest.raises(RuntimeError):   # N not a multiple of 8
        ops.gemm(a, torch.zeros(12, 64, device=DEV, dtype=torch.bfloat16),
                 torch.zeros(128, 12, device=DEV, dtype=torch.bfloat16), False, False, None, None,
                 False, 1.0, 0)


def attention_reference(qkv, B, S, hq, hkv, mask, scale):
    D = 128
    x = qkv.float().view(B, S, hq + 2 * hkv, D).clone().requires_grad_(True)
    q = x[:, :, :hq].transpose(1, 2)
    k = x[:, :, hq:hq + hkv].transpose(1, 2).repeat_interleave(hq // hkv, 1)
    v = x[:, :, hq + hkv:].transpose(1, 2).repeat_interleave(hq // hkv, 1)
    scores = q @ k.transpose(-1, -2) * scale
    allow = torch.ones(S, S, dtype=torch.bool, device=DEV).tril()[None, None].expand(B, 1, S, S)
    if mask is not None:
        allow = allow & mask.bool()[:, None, None, :]
    scores = scores.masked_fill(~allow, float("-inf"))
    dead = ~allow.any(-1, keepdim=True)
    probs = torch.softmax(scores.masked_fill(dead, 0), -1).masked_fill(dead, 0)
    return x, (probs @ v).transpose(1, 2).reshape(B * S, hq * D)


@pytest.mark.parametrize("B,S,hq,hkv,masked", [(1, 128, 2, 1, False), (2, 512, 12, 2, False),
                                               (2, 384, 4, 2, True), (1, 200, 2, 1, False),
                                               (1, 1024, 4, 1, False),
                                               (1, 2048, 7, 1, False),     # 7B, TP 4: 7 / 1 local heads
                                               (3, 256, 4, 2, "padded")])  # one fully padded sample
def test_attention_forward_backward(ops, B, S, hq, hkv, masked):
    torch.manual_seed(0)
    D, W = 128, (hq + 2 * hkv) * 128
    qkv = (torch.randn(B * S, W, device=DEV) * 0.5).bfloat16()
    mask = None
    if masked:
        mask = torch.ones(B, S, dtype=torch.uint8, device=DEV)
        mask[0, : S // 3] = 0
        mask[-1, S // 2:] = 0
        if masked == "padded":
            mask[1] = 0                      # nothing to attend to: output rows and grads are 0
    scale = 1 / math.sqrt(D)
    out = torch.zeros(B * S, hq * D, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros(B, hq, S, device=DEV)
    ops.attention_fwd(qkv, out, lse, mask, B, S, hq, hkv, scale)
    x, ref = attention_reference(qkv, B, S, hq, hkv, mask, scale)
    assert rel(out, ref) < 5e-3
    # elementwise on the rows where a Frobenius ratio hides a wrong element: the first and last
    # query block, and every row of a masked sample
    edge = torch.cat([torch.arange(0, min(S, 130)), torch.arange(B * S - 130, B * S)]).to(DEV)
    torch.testing.assert_close(out[edge].float(), ref[edge].detach(), atol=2e-2, rtol=2e-2)
    if masked:
        torch.testing.assert_close(out.float(), ref.detach(), atol=2e-2, rtol=2e-2)
    if masked == "padded":
        assert not out.view(B, S, -1)[1].any()
    dout = (torch.randn(B * S, hq * D, device=DEV) * 0.5).bfloat16()
    ref.backward(dout.float())
    want = x.grad.view(B * S, W)
    delta = torch.zeros(B, hq, S, device=DEV)
    dqkv = torch.zeros(B * S, W, device=DEV, dtype=torch.bfloat16)
    ops.attention_bwd(qkv, out, dout, lse, delta, dqkv, delta, mask, B, S, hq, hkv, scale)
    for lo, hi in ((0, hq * D), (hq * D, (hq + hkv) * D), ((hq + hkv) * D, W)):
        assert rel(dqkv[:, lo:hi], want[:, lo:hi]) < 6e-3
    torch.testing.assert_close(dqkv[edge].float(), want[edge], atol=6e-2, rtol=5e-2)
    if masked == "padded":
        assert not dqkv.view(B, S, -1)[1].any()
    if masked:
        # the packed form of the mask (one bit per key) drives the same kernels to the same bits
        bits = torch.empty(B, 4 * ((S + 127) // 128), device=DEV, dtype=torch.int32)
        ops.pack_key_mask(mask, bits)
        out_b, lse_b = torch.zeros_like(out), torch.zeros_like(lse)
        ops.attention_fwd(qkv, out_b, lse_b, bits, B, S, hq, hkv, scale)
        assert torch.equal(out_b, out) and torch.equal(lse_b, lse)
        dqkv_b = torch.zeros_like(dqkv)
        ops.attention_bwd(qkv, out, dout, lse, delta, dqkv_b, delta, bits, B, S, hq, hkv, scale)
        assert torch.equal(dqkv_b, dqkv)
        word = bits.view(B, -1)[0, 0].item() & 0xFFFFFFFF
        assert word == sum(int(mask[0, i].item() != 0) << i for i in range(32))
    # with a scratch large enough the query-head group is split over several dK/dV CTAs per kv
    # head and the fp32 partial planes are added in a fixed order: same result, twice
    scratch = torch.full(((hq // hkv) * B * S * 2 * hkv * D,), float("nan"), device=DEV)
    split = [torch.zeros_like(dqkv), torch.zeros_like(dqkv)]
    for target in split:
        ops.attention_bwd(qkv, out, dout, lse, delta, target, scratch, mask, B, S, hq, hkv, scale)
    assert torch.equal(split[0], split[1])
    for lo, hi in ((0, hq * D), (hq * D, (hq + hkv) * D), ((hq + hkv) * D, W)):
        assert rel(split[0][:, lo:hi], want[:, lo:hi]) < 6e-3


def test_rmsnorm_rope_swiglu(ops):
    torch.manual_seed(1)
    T, H = 300, 1536
    x, w = torch.randn(T, H, device=DEV), torch.randn(H, device=DEV)
    y = torch.empty(T, H, device=DEV, dtype=torch.bfloat16)
    inv = torch.empty(T, device=DEV)
    ops.rmsnorm_fwd(x, w, y, inv, 1e-6)
    y_ref = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + 1e-6) * w
    assert rel(y, y_ref) < 4e-3
    close_on_edges(y, y_ref, atol=2e-2, rtol=1e-2)
    dy, dres = torch.randn(T, H, device=DEV), torch.randn(T, H, device=DEV)
    dx, part = torch.empty_like(x), torch.empty(592, H, device=DEV)
    ops.rmsnorm_bwd(dy, x, w, inv, dres, dx, part)
    dw = torch.empty(H, device=DEV)
    ops.colsum_f32(part, dw, False)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    (xr * torch.rsqrt(xr.square().mean(-1, keepdim=True) + 1e-6) * wr).backward(dy)
    assert rel(dx, xr.grad + dres) < 1e-5 and rel(dw, wr.grad) < 1e-5
    close_on_edges(dx, xr.grad + dres, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(dw, wr.grad, atol=2e-3, rtol=1e-4)
    hq, hkv, d, S = 12, 2, 128, 256
    rows = 2 * S
    qkv = torch.randn(rows, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    ang = torch.arange(S, device=DEV).float()[:, None] * (1e6 ** (-torch.arange(0, d, 2, device=DEV).float() / d))[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    before = qkv.clone()
    ops.rope(qkv, cos, sin, None, S, hq, hkv, d, False)
    t = before[:, :hq * d].float().view(rows, hq, d)
    c = torch.cat([cos, cos], -1).repeat(2, 1)[:, None]
    s = torch.cat([sin, sin], -1).repeat(2, 1)[:, None]
    want = (t * c + torch.cat([-t[..., d // 2:], t[..., :d // 2]], -1) * s).reshape(rows, hq * d)
    assert rel(qkv[:, :hq * d], want) < 4e-3
    close_on_edges(qkv[:, :hq * d], want, atol=3e-2, rtol=1e-2)
    assert torch.equal(qkv[:, (hq + hkv) * d:], before[:, (hq + hkv) * d:])
    ops.rope(qkv, cos, sin, None, S, hq, hkv, d, True)
    assert rel(qkv, before) < 4e-3
    inter = 8960
    gu = torch.randn(T, 2 * inter, device=DEV).bfloat16()
    h = torch.empty(T, inter, device=DEV, dtype=torch.bfloat16)
    ops.swiglu_fwd(gu, h)
    g, u = gu[:, :inter].float(), gu[:, inter:].float()
    assert rel(h, torch.nn.functional.silu(g) * u) < 6e-3
    close_on_edges(h, torch.nn.functional.silu(g).bfloat16().float() * u, atol=2e-2, rtol=1e-2)
    dh, dgu = torch.randn(T, inter, device=DEV).bfloat16(), torch.empty_like(gu)
    ops.swiglu_bwd(dh, gu, dgu)
    gr, ur = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
    (torch.nn.functional.silu(gr) * ur).backward(dh.float())
    assert rel(dgu[:, :inter], gr.grad) < 4e-3 and rel(dgu[:, inter:], ur.grad) < 4e-3
    close_on_edges(dgu[:, :inter], gr.grad, atol=3e-2, rtol=1.5e-2)
    close_on_edges(dgu[:, inter:], ur.grad, atol=3e-2, rtol=1.5e-2)


def test_cross_entropy_and_column_sums(ops):
    torch.manual_seed(2)
    R, V = 200, 151936
    logits = (torch.randn(R, V, device=DEV) * 2).bfloat16()
    labels = torch.randint(0, V, (R,), device=DEV)
    labels[::7] = -100
    lse, rows, total = torch.empty(R, device=DEV), torch.empty(R, device=DEV), torch.zeros(1, device=DEV)
    ops.ce_fwd(logits, labels, lse, rows)
    ops.sum_f32(rows, total, False)
    lf = logits.float().clone().requires_grad_(True)
    want = torch.nn.functional.cross_entropy(lf, labels, ignore_index=-100, reduction="sum")
    assert abs(total.item() - want.item()) / want.item() < 1e-5
    want.backward()
    ops.ce_bwd(logits, labels, lse, torch.full((1,), 0.5, device=DEV))
    assert rel(logits, lf.grad * 0.5) < 5e-3
    close_on_edges(logits, lf.grad * 0.5, atol=2e-3, rtol=1.5e-2)
    ignored = labels.eq(-100)
    assert not logits[ignored].any()                    # ignored rows have a zero gradient
    hit = logits[~ignored].float().gather(1, labels[~ignored][:, None])
    torch.testing.assert_close(hit, (lf.grad * 0.5)[~ignored].gather(1, labels[~ignored][:, None]),
                               atol=2e-3, rtol=1.5e-2)     # the "- onehot" element of every row
    x = torch.randn(777, 2048, device=DEV).bfloat16()
    out, scratch = torch.empty(2048, device=DEV), torch.empty(64, 2048, device=DEV)
    ops.colsum_bf16(x, out, False, scratch)
    assert rel(out, x.float().sum(0)) < 1e-5
    torch.testing.assert_close(out, x.float().sum(0), atol=1e-3, rtol=1e-5)


def test_optimizer_and_gradient_check(ops):
    torch.manual_seed(3)
    n = 1000003
    p, g = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    ref = torch.nn.Parameter(p.clone())
    ref.grad = g.clone()
    opt = torch.optim.AdamW([ref], lr=1e-3)
    for step in (1, 2, 3):
        opt.step()
        ops.adamw(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1 - 0.9 ** step, 1 - 0.999 ** step, 1.0)
    assert (p - ref.data).abs().max().item() < 3e-6
    flags = torch.zeros(2, device=DEV, dtype=torch.int32)
    grad = torch.zeros(10000, device=DEV)
    pads = torch.tensor([100, 200], device=DEV)
    ops.grad_check(grad, pads, flags)
    assert flags.tolist() == [0, 0]
    grad[150] = 1.0
    ops.grad_check(grad, pads, flags)
    assert flags.tolist() == [0, 1]
    flags.zero_()
    grad[150], grad[5000] = 0, float("nan")
    ops.grad_check(grad, pads, flags)
    assert flags.tolist() == [1, 0]


def test_shard_gather_and_reduce_scatter_with_emulated_ranks(ops):
    """Degree-2 tables over two buffers of one GPU: the kernels only use plain loads, so the
    rank dimension can be emulated without a second device."""
    F = 2
    numels = [1536 * 2048, 1536, 2048 * 3 + 1, 1000]
    segs, shard_off, full_off = [], 0, 0
    for i, n in enumerate(numels):
        q = -(-n // F)
        segs.append([shard_off, q, n, full_off, 1 if i in (1, 3) else 0])
        shard_off += -(-q // 8) * 8
        full_off += -(-n // 8) * 8
    table = torch.tensor(segs, dtype=torch.int64)
    fulls = [torch.randn(n, device=DEV) for n in numels]
    shards = [torch.zeros(shard_off, device=DEV) for _ in range(F)]
    for (so, q, n, fo, k), f in zip(segs, fulls):
        for r in range(F):
            keep = max(0, min(q, n - r * q))
            shards[r][so:so + keep] = f[r * q:r * q + keep]
    fb, ff = torch.zeros(full_off, device=DEV, dtype=torch.bfloat16), torch.zeros(full_off, device=DEV)
    ops.gather_params([s.data_ptr() for s in shards], table, fb, ff)
    for (so, q, n, fo, k), f in zip(segs, fulls):
        got = ff[fo:fo + n] if k else fb[fo:fo + n].float()
        assert torch.equal(got, f if k else f.bfloat16().float())
    # the same gather from the owners' bf16 shadow arenas: half the bytes, identical bits
    shadows = [s.bfloat16() for s in shards]
    fb2, ff2 = torch.zeros_like(fb), torch.zeros_like(ff)
    ops.gather_params([s.data_ptr() for s in shards], table, fb2, ff2, [s.data_ptr() for s in shadows])
    assert torch.equal(fb2, fb) and torch.equal(ff2, ff)
    grads = [torch.randn(full_off, device=DEV) for _ in range(F)]
    for r in range(F):
        gs = torch.ones(shard_off, device=DEV)
        p, m, v = torch.randn(shard_off, device=DEV), torch.zeros(shard_off, device=DEV), torch.zeros(shard_off, device=DEV)
        p0 = p.clone()
        shadow = torch.zeros(shard_off, device=DEV, dtype=torch.bfloat16)
        ops.reduce_scatter_adamw([t.data_ptr() for t in grads], r, table, gs, p, m, v, 0.5, True,
                                 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, None, 1, 0, 1.0, shadow)
        for (so, q, n, fo, k) in segs:
            assert torch.equal(shadow[so:so + q], p[so:so + q].bfloat16())
        for (so, q, n, fo, k) in segs:
            keep = max(0, min(q, n - r * q))
            want = 1 + 0.5 * sum(t[fo + r * q:fo + r * q + keep] for t in grads)
            torch.testing.assert_close(gs[so:so + keep], want, atol=1e-6, rtol=1e-6)
            assert (gs[so + keep:so + q] == 1).all()      # accumulate adds exact zero in the padding
            ref = torch.nn.Parameter(p0[so:so + keep].clone())
            ref.grad = want.clone()
            torch.optim.AdamW([ref], lr=1e-3).step()
            torch.testing.assert_close(p[so:so + keep], ref.data, atol=2e-6, rtol=2e-6)


def test_bounded_peer_wait_reports_instead_of_hanging(ops):
    """A flag nobody sets: the barrier kernel gives up once its *time* budget is spent and
    records a status block; the context stays usable.  Budgets here are a few milliseconds."""
    import time

    from shardtrain_b200 import ops as module

    budget_us = 5000
    pad_a = torch.zeros(64, device=DEV, dtype=torch.int32)
    pad_b = torch.zeros(64, device=DEV, dtype=torch.int32)
    ops.peer_barrier([pad_a.data_ptr()], 0, 1, 0, budget_us)
    torch.cuda.synchronize()
    assert ops.status_read() == 0
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    ops.peer_barrier([pad_a.data_ptr(), pad_b.data_ptr()], 0, 5, 1, budget_us)   # "peer 1" never signals
    end.record()
    torch.cuda.synchronize()
    waited_ms = begin.elapsed_time(end)
    assert 0.5 * budget_us / 1e3 <= waited_ms <= 10 * budget_us / 1e3, waited_ms
    # with the failure on record, a second barrier on an unset flag returns without spinning its
    # budget, and work queued behind the failure is skipped instead of running on stale data
    x = torch.randn(256, 128, device=DEV).bfloat16()
    w = torch.randn(256, 128, device=DEV).bfloat16()
    out = torch.full((256, 256), 7.0, device=DEV, dtype=torch.bfloat16)
    begin.record()
    ops.peer_barrier([pad_a.data_ptr(), pad_b.data_ptr()], 0, 6, 1, 1_000_000)    # 1 s budget
    ops.gemm(x, w, out, False, False, None, None, False, 1.0, 0)
    end.record()
    torch.cuda.synchronize()
    assert begin.elapsed_time(end) < 100.0            # nowhere near the 1 s budget
    assert bool((out == 7.0).all())                    # the GEMM did not run
    with pytest.raises(RuntimeError, match="peer flag wait expired") as info:
        module.check_status("test")
    # who was silent, which epoch was awaited, what was last seen
    assert "group member 1 silent: waited for epoch 5, last saw 0" in str(info.value)
    assert ops.status_read() == 0
    assert torch.ones(4, device=DEV).sum().item() == 4
    ops.gemm(x, w, out, False, False, None, None, False, 1.0, 0)     # status cleared: runs again
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), x.float() @ w.float().t(), atol=0.5, rtol=2e-2)
    # the small all-reduce has the same bounded wait; a single member never waits
    pads, inbox = [pad_a.data_ptr(), pad_b.data_ptr()], torch.zeros(2, 2 * 8 * 16, device=DEV,
                                                                   dtype=torch.float64)
    values, out = torch.tensor([1.5, 2.0], device=DEV, dtype=torch.float64), torch.zeros(2, device=DEV, dtype=torch.float64)
    t0 = time.perf_counter()
    ops.peer_allreduce_small(pads, [inbox[0].data_ptr(), inbox[1].data_ptr()], 0, 9, 6, values, out, 0, budget_us)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    with pytest.raises(RuntimeError, match="waited for epoch 9"):
        module.check_status("test")
    ops.peer_allreduce_small(pads[:1], [inbox[0].data_ptr()], 0, 10, 6, values, out, 0, budget_us)
    torch.cuda.synchronize()
    module.check_status("test")
    assert out.tolist() == [1.5, 2.0]


@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_scatter_epilogue_routes_rows_to_their_sequence_owner(ops, b_mn):
    """Row-parallel GEMM -> sequence reduce-scatter: the epilogue writes row b*S + s into the
    buffer of owner s // (S/T) at row b*(S/T) + s % (S/T).  The owners' buffers are emulated by
    local tensors (plain stores, nothing waits on a peer)."""
    B, S, T, N, K = 3, 256, 2, 512, 384
    a = torch.randn(B * S, K, device=DEV).bfloat16()
    w = (torch.randn(K, N, device=DEV) if b_mn else torch.randn(N, K, device=DEV)).bfloat16()
    dest = [torch.full((B * S // T, N), float("nan"), device=DEV) for _ in range(T)]
    ops.gemm_scatter(a, w, [d.data_ptr() for d in dest], S, False, b_mn, 0)
    want = a.float() @ (w.float() if b_mn else w.float().t())
    want = want.view(B, T, S // T, N)
    for t in range(T):
        torch.testing.assert_close(dest[t].view(B, S // T, N), want[:, t], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("with_norm", [True, False])
def test_slot_sum_rmsnorm(ops, with_norm):
    rows, cols, T = 300, 1536, 3
    slots = torch.randn(T, rows, cols, device=DEV)
    residual = torch.randn(rows, cols, device=DEV)
    out = torch.empty(rows, cols, device=DEV)
    if with_norm:
        w = torch.randn(cols, device=DEV)
        y = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
        inv = torch.empty(rows, device=DEV)
        ops.slot_sum_rmsnorm(slots, residual, out, w, y, inv, 1e-6)
    else:
        ops.slot_sum_rmsnorm(slots, None, out, None, None, None, 0.0)
    want = slots.sum(0) + (residual if with_norm else 0)
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)
    if with_norm:
        r = torch.rsqrt(want.pow(2).mean(-1) + 1e-6)
        torch.testing.assert_close(inv, r, atol=1e-5, rtol=1e-5)
        assert rel(y, want * r[:, None] * w) < 5e-3


def test_reduce_scatter_sums_replicated_segments_over_the_whole_mesh(ops):
    """F=2 x T=2 mesh emulated on one GPU: a TP-split parameter is reduced over the two ranks
    of its TP coordinate, a TP-replicated one (table flag 2) over all four, with its own scale;
    both TP replicas must end with bit-identical replicated shards."""
    F, T = 2, 2
    numels, replicated = [4096 * 3, 1000], [False, True]
    segs, shard_off, full_off = [], 0, 0
    for n, rep in zip(numels, replicated):
        q = -(-n // F)
        segs.append([shard_off, q, n, full_off, 2 if rep else 0])
        shard_off += -(-q // 4) * 4
        full_off += -(-n // 4) * 4
    table = torch.tensor(segs, dtype=torch.int64)
    slots = [torch.randn(full_off, device=DEV) for _ in range(F * T)]     # index f * T + t
    ptrs = [s.data_ptr() for s in slots]
    results = {}
    for f in range(F):
        for t in range(T):
            gs = torch.zeros(shard_off, device=DEV)
            flags = torch.zeros(2, device=DEV, dtype=torch.int32)
            ops.reduce_scatter(ptrs, f, table, gs, 1.0 / F, False, flags, T, t, 0.25)
            results[f, t] = gs
            assert flags.tolist() == [0, 0]
            for (so, q, n, fo, flag) in segs:
                keep = max(0, min(q, n - f * q))
                piece = slice(fo + f * q, fo + f * q + keep)
                if flag:
                    want = 0.25 * sum(s[piece] for s in slots)
                else:
                    want = sum(slots[g * T + t][piece] for g in range(F)) / F
                torch.testing.assert_close(gs[so:so + keep], want, atol=1e-6, rtol=1e-6)
    so, q = segs[1][0], segs[1][1]
    for f in range(F):
        assert torch.equal(results[f, 0][so:so + q], results[f, 1][so:so + q])


@pytest.mark.parametrize("T,B,sl,cols", [(2, 3, 64, 512), (4, 1, 40, 1536), (1, 2, 7, 128)])
def test_sequence_gather_and_pull_reduce_scatter(ops, T, B, sl, cols):
    """Sequence all-gather / reduce-scatter kernels with the peers emulated by local tensors."""
    parts = [torch.randn(B, sl, cols, device=DEV).bfloat16() for _ in range(T)]
    out = torch.empty(B * T * sl, cols, device=DEV, dtype=torch.bfloat16)
    ops.seq_gather([p.data_ptr() for p in parts], out, B, sl, cols * 2)
    assert torch.equal(out.view(B, T * sl, cols), torch.cat(parts, dim=1))
    partials = [torch.randn(B, T * sl, cols, device=DEV) for _ in range(T)]
    residual = torch.randn(B, sl, cols, device=DEV)
    for rank in range(T):
        got = torch.empty(B, sl, cols, device=DEV)
        ops.seq_reduce_scatter([p.data_ptr() for p in partials], rank, residual, got, B, sl)
        want = residual + sum(p[:, rank * sl:(rank + 1) * sl] for p in partials)
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("M,inter,K", [(512, 1024, 256), (300, 8960, 1536), (4096, 328, 192)])
def test_gate_up_gemm_with_swiglu_epilogue(ops, M, inter, K):
    """One kernel for gu = x @ [Wg; Wu]^T and h = bf16(silu(gate)) * up, against the separate
    GEMM + SwiGLU kernels (bit-identical) and an fp32 reference."""
    torch.manual_seed(5)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * inter, K, device=DEV) / math.sqrt(K)).bfloat16()
    gu, h = torch.empty(M, 2 * inter, device=DEV, dtype=torch.bfloat16), torch.empty(M, inter, device=DEV, dtype=torch.bfloat16)
    ops.gemm_swiglu(x, w, gu, h)
    gu2, h2 = torch.empty_like(gu), torch.empty_like(h)
    ops.gemm(x, w, gu2, False, False, None, None, False, 1.0, 256, 1)
    ops.swiglu_fwd(gu2, h2)
    assert torch.equal(gu, gu2) and torch.equal(h, h2)
    ref = x.float() @ w.float().t()
    assert rel(gu, ref) < 5e-3
    assert rel(h, torch.nn.functional.silu(ref[:, :inter]) * ref[:, inter:]) < 1e-2


def test_gemm_broadcast_epilogue_writes_every_row_to_every_destination(ops):
    """All-reduce push of tensor parallelism without SP: the fp32 result goes, row for row, into
    each member's receive slot (local tensors stand in for the members)."""
    from shardtrain_b200 import ops as module

    M, N, K, T = 640, 512, 320, 3
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    want = a.float() @ w.float().t()
    dest = [torch.full((M, N), float("nan"), device=DEV) for _ in range(T)]
    module.load().gemm_broadcast(a, w, [d.data_ptr() for d in dest], False)
    for d in dest:
        torch.testing.assert_close(d, want, atol=2e-2, rtol=2e-2)
        assert torch.equal(d, dest[0])


def _shard_arenas(weights, degree, fp32):
    """Cut each [rows, K] parameter into `degree` flat shards (q = ceil(numel / F), zero padded)
    and lay the shards of all parameters out one after another in `degree` emulated rank arenas.
    Returns (arenas, segment table rows [shard_off, q, numel, full_off, 0])."""
    offsets, table, cursor, full_cursor = [], [], 0, 0
    for w in weights:
        numel = w.numel()
        q = -(-numel // degree)
        table.append([cursor, q, numel, full_cursor, 0])
        offsets.append((cursor, q))
        cursor += -(-q // 8) * 8 if q % 8 == 0 else q     # keep odd layouts odd on purpose
        full_cursor += -(-numel // 8) * 8
    dtype = torch.float32 if fp32 else torch.bfloat16
    arenas = [torch.zeros(cursor + 8, device=DEV, dtype=dtype) for _ in range(degree)]
    for w, (off, q) in zip(weights, offsets):
        flat = w.reshape(-1).to(dtype)
        for r in range(degree):
            piece = flat[r * q:(r + 1) * q]
            arenas[r][off:off + piece.numel()] = piece
    return arenas, torch.tensor(table, dtype=torch.int64), full_cursor


AG_CASES = [
    # M, K, rows of each parameter, F, fp32 wire, bias, force_bn
    (512, 1536, (1536, 256, 256), 8, False, True, 0),       # q|k|v of the 1.5B layer
    (512, 1536, (1536, 256, 256), 8, False, True, 128),
    (1024, 512, (512, 128, 128), 4, False, False, 64),      # eight row tiles, one pass
    (1100, 256, (384,), 2, False, True, 128),               # three passes: later ones read `full`
    (300, 392, (72, 40), 5, False, True, 0),                # K tail, shards that end mid-row (odd q)
    (200, 264, (104,), 7, True, False, 0),                  # fp32 on the wire, unaligned shards
    (512, 1536, (1536, 256, 256), 8, True, True, 0),        # fp32 on the wire, aligned
]


@pytest.mark.parametrize("case", AG_CASES, ids=[f"m{c[0]}k{c[1]}f{c[3]}{'w32' if c[4] else ''}bn{c[6]}" for c in AG_CASES])
def test_allgather_fused_into_gemm_with_emulated_ranks(ops, case):
    """out = A @ W^T where W's rows are pulled inside the GEMM from the F ranks' shard arenas
    (local tensors stand in for the peers' memory; the kernel only reads them).  Checked
    elementwise against the FP32 product, and the by-product copy of W against W itself."""
    M, K, rows, degree, fp32, with_bias, bn = case
    torch.manual_seed(1)
    weights = [(torch.randn(r, K, device=DEV) * 0.5).bfloat16() for r in rows]
    W = torch.cat(weights)
    N = W.shape[0]
    a = torch.randn(M, K, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV) if with_bias else None
    arenas, table, full_numel = _shard_arenas(weights, degree, fp32)
    full = torch.full((full_numel,), float("nan"), device=DEV, dtype=torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_allgather(a, out, bias, [t.data_ptr() for t in arenas], fp32, table, full, None, bn)
    ref = a.float() @ W.float().t()
    if with_bias:
        ref = ref + bias
    torch.testing.assert_close(out.float(), ref, atol=0.25, rtol=2e-2)
    assert rel(out, ref) < 4e-3
    # edge rows / columns elementwise (ragged tiles, last row tile)
    torch.testing.assert_close(out[-3:].float(), ref[-3:], atol=0.25, rtol=2e-2)
    torch.testing.assert_close(out[:, -5:].float(), ref[:, -5:], atol=0.25, rtol=2e-2)
    # the pulled rows were mirrored into the local full buffer, bit for bit
    cursor = 0
    for w in weights:
        assert torch.equal(full[cursor:cursor + w.numel()].view_as(w), w)
        cursor += -(-w.numel() // 8) * 8
    # same result as the two-kernel path (gather, then GEMM): bit-identical accumulation order
    two = torch.empty_like(out)
    ops.gemm(a, W, two, False, False, bias, None, False, 1.0, 0)
    assert rel(out, two) < 2e-3


@pytest.mark.parametrize("M,inter,K,degree", [(512, 896, 1536, 8), (300, 328, 256, 4), (1024, 256, 512, 2)])
def test_allgather_fused_into_gate_up_gemm_with_swiglu(ops, M, inter, K, degree):
    """Gated variant: W = gate|up pulled from the shard arenas, SwiGLU in the epilogue; gu and
    h agree with the local gated GEMM on the gathered weight (each tile walks K from its own
    starting block, so the fp32 sums differ in the last bits, not more)."""
    torch.manual_seed(2)
    gate = (torch.randn(inter, K, device=DEV) * 0.3).bfloat16()
    up = (torch.randn(inter, K, device=DEV) * 0.3).bfloat16()
    a = torch.randn(M, K, device=DEV).bfloat16()
    arenas, table, full_numel = _shard_arenas([gate, up], degree, False)
    full = torch.zeros(full_numel, device=DEV, dtype=torch.bfloat16)
    gu = torch.full((M, 2 * inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    h = torch.full((M, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_allgather(a, gu, None, [t.data_ptr() for t in arenas], False, table, full, h, 0)
    w_gu = torch.cat([gate, up])
    ref_gu = torch.empty_like(gu)
    ref_h = torch.empty_like(h)
    ops.gemm_swiglu(a, w_gu, ref_gu, ref_h)
    torch.testing.assert_close(gu.float(), ref_gu.float(), atol=0.07, rtol=1.6e-2)
    torch.testing.assert_close(h.float(), ref_h.float(), atol=0.07, rtol=1.6e-2)
    assert rel(gu, ref_gu) < 1e-3 and rel(h, ref_h) < 2e-3
    want = a.float() @ w_gu.float().t()
    torch.testing.assert_close(gu.float(), want, atol=0.25, rtol=2e-2)
    g32, u32 = gu[:, :inter].float(), gu[:, inter:].float()
    torch.testing.assert_close(h.float(), torch.nn.functional.silu(g32).bfloat16().float() * u32,
                               atol=0.05, rtol=2e-2)
    assert torch.equal(full[:gate.numel()].view_as(gate), gate)      # the by-product copy


def test_allgather_gemm_rejects_bad_arguments(ops):
    a = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    arenas, table, full_numel = _shard_arenas([w], 2, False)
    out = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    ptrs = [t.data_ptr() for t in arenas]
    with pytest.raises(RuntimeError):        # rows of the table do not add up to N
        ops.gemm_allgather(a, torch.zeros(128, 72, device=DEV, dtype=torch.bfloat16), None, ptrs,
                           False, table, None, None, 0)
    with pytest.raises(RuntimeError):        # more row tiles than TMEM accumulators, no `full`
        big = torch.zeros(1100, 64, device=DEV, dtype=torch.bfloat16)
        ops.gemm_allgather(big, torch.zeros(1100, 64, device=DEV, dtype=torch.bfloat16), None, ptrs,
                           False, table, None, None, 128)
    with pytest.raises(RuntimeError):        # misaligned arena
        ops.gemm_allgather(a, out, None, [ptrs[0] + 2, ptrs[1]], False, table, None, None, 0)
    torch.cuda.synchronize()


@pytest.mark.parametrize("T,B,sl,K,N,b_mn", [(2, 2, 256, 512, 384, False), (4, 1, 96, 264, 520, False),
                                             (8, 3, 64, 1536, 2048, False), (2, 2, 128, 256, 512, True)])
def test_sequence_gather_fused_into_gemm_with_emulated_peers(ops, T, B, sl, K, N, b_mn):
    """A is the sequence all-gather of T ranks' [B, sl, K] slices, pulled by the GEMM itself
    (local tensors stand in for the peers' buffers).  The result and the gathered operand the
    kernel leaves behind are checked against the FP32 product / the plain concatenation."""
    torch.manual_seed(3)
    slices = [torch.randn(B * sl, K, device=DEV).bfloat16() for _ in range(T)]
    w = (torch.randn(K, N, device=DEV) if b_mn else torch.randn(N, K, device=DEV)).bfloat16()
    bias = torch.randn(N, device=DEV)
    M = B * T * sl
    a_dst = torch.full((M, K), float("nan"), device=DEV, dtype=torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    for _ in range(2):          # a second launch reuses the flag buffer with a new epoch
        a_dst.fill_(float("nan"))
        ops.gemm_seq_pull(a_dst, w, out, b_mn, bias, [s.data_ptr() for s in slices], B, sl, 0)
    gathered = torch.stack([s.view(B, sl, K) for s in slices], dim=1).reshape(M, K)
    assert torch.equal(a_dst, gathered)
    ref = gathered.float() @ (w.float() if b_mn else w.float().t()) + bias
    torch.testing.assert_close(out.float(), ref, atol=0.5, rtol=2e-2)
    assert rel(out, ref) < 4e-3
    two = torch.empty_like(out)
    ops.gemm(gathered, w, two, False, b_mn, bias, None, False, 1.0, 0)
    assert torch.equal(out, two)      # same tiles, same accumulation order as the plain GEMM


@pytest.mark.parametrize("degree", [1, 2, 4, 8])
def test_packing_kernels_of_the_library_collective_path_match_the_torch_path(ops, degree):
    """Single-launch unpack of the rank-major gather buffer and pack of the destination-major
    gradient buffer (fp32, CUDA) against the per-parameter torch copies on the CPU: equal bits,
    zero padding, odd sizes, a non-contiguous gradient."""
    from shardtrain_b200.runtime.layout import ParameterSpec, copy_out, offsets, pack_gradients, shard_of

    torch.manual_seed(degree)
    shapes = [(3, 5), (7,), (2, 2, 3), (1,), (1031, 67), (8, 8)]
    specs = [ParameterSpec.create(f"p{i}", 0, torch.empty(s), s, "column", degree)
             for i, s in enumerate(shapes)]
    tensors = [torch.randn(s) for s in shapes]
    starts, slot = offsets(specs)
    storage = torch.zeros(degree * slot)
    for rank in range(degree):
        for t, spec, start in zip(tensors, specs, starts):
            storage[rank * slot + start: rank * slot + start + spec.fsdp_shard_numel] = shard_of(t, spec, rank)
    before = int(ops.launch_count())
    got = copy_out(storage.to(DEV), specs, degree)
    assert int(ops.launch_count()) == before + 1              # one kernel for the whole unit
    want = copy_out(storage, specs, degree)
    for spec in specs:
        assert got[spec.param_id].shape == want[spec.param_id].shape
        assert torch.equal(got[spec.param_id].cpu(), want[spec.param_id])
    grads_gpu = [t.to(DEV) for t in tensors]
    grads_gpu[4] = tensors[4].t().contiguous().to(DEV).t()    # same values, column-major storage
    assert not grads_gpu[4].is_contiguous()
    packed = pack_gradients(grads_gpu, specs, degree)
    assert torch.equal(packed.cpu(), pack_gradients(tensors, specs, degree))
