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
    too_wide = torch.zeros(2, 8192 + 2, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8192 + 2, device="cuda")
    assert fn(too_wide.data_ptr(), too_wide.stride(0), out.data_ptr(), 2, 8192 + 2, 0, stream) == -1
    assert fn(None, 8, out.data_ptr(), 2, 8, 0, stream) == -1
    assert fn(too_wide.data_ptr(), 8, out.data_ptr(), 2, 7, 0, stream) == -1
