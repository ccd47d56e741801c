"""The allocation-free column-sum entry point, called through its exported C symbol.

Some embedders of the library may not call cudaMalloc while they run (a foreign stream capture
in progress, a fixed-budget real-time loop, a process that pre-partitioned the device), so this
entry point keeps its workspace inside the library.  The test checks it against the regular op,
which takes the workspace from the caller, on two consecutive calls (the shared workspace keeps
the first call's partial sums, the second must not be affected by them).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_colsum_matches_the_regular_op_twice_in_a_row():
    from shardtrain_b200 import ops

    namespace = ops.load()
    lib = ctypes.CDLL(ops.extension_path())
    fn = lib.stb_colsum_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, cols, scale in ((777, 2048, 1.0), (4096, 1536, 3.0)):
        x = (torch.randn(rows, cols, device="cuda") * scale).bfloat16()
        want = torch.empty(cols, device="cuda")
        namespace.colsum_bf16(x, want, False, torch.empty(64, cols, device="cuda"))
        got = torch.full((cols,), 7.0, device="cuda")
        before = torch.cuda.memory_allocated()
        code = fn(x.data_ptr(), x.stride(0), got.data_ptr(), rows, cols, 0, stream)
        assert code == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        rel = ((got - want).norm() / want.norm()).item()
        assert rel < 1e-5, rel
        # accumulate on top of the previous result
        assert fn(x.data_ptr(), x.stride(0), got.data_ptr(), rows, cols, 1, stream) == 0
        torch.cuda.synchronize()
        assert ((got - 2 * want).norm() / (2 * want).norm()).item() < 1e-5
    # strided rows (ldx > cols), fewer rows than partial-sum rows, and a side stream; the free
    # bytes the driver reports must not move (a raw cudaMalloc would not show in torch's counters)
    side = torch.cuda.Stream()
    wide = (torch.randn(37, 1024, device="cuda")).bfloat16()
    view = wide[:, 128:640]                      # ldx 1024, cols 512, 4-byte aligned start
    want = view.float().sum(0)
    got = torch.empty(512, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    with torch.cuda.stream(side):
        assert fn(view.data_ptr(), view.stride(0), got.data_ptr(), 37, 512, 0, side.cuda_stream) == 0
    side.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-4)
    # a view starting at an odd element offset is refused on the host, nothing is launched
    odd = wide[:, 1:513]
    assert odd.data_ptr() % 4 == 2
    assert fn(odd.data_ptr(), odd.stride(0), got.data_ptr(), 37, 512, 0, stream) == -1
    assert fn(view.data_ptr(), view.stride(0), got.data_ptr() + 2, 37, 510, 0, stream) == -1
    assert fn(view.data_ptr(), 1023, got.data_ptr(), 37, 512, 0, stream) == -1
    too_wide = torch.zeros(2, 8192 + 2, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8192 + 2, device="cuda")
    assert fn(too_wide.data_ptr(), too_wide.stride(0), out.data_ptr(), 2, 8192 + 2, 0, stream) == -1
    assert fn(None, 8, out.data_ptr(), 2, 8, 0, stream) == -1
    assert fn(too_wide.data_ptr(), 8, out.data_ptr(), 2, 7, 0, stream) == -1
