"""The allocation-free top-k entry point, called through its exported C symbol.

Some callers cannot allocate device memory (their own pool owns the GPU, or they run
where an allocator lock must not be taken, or they are plain C programs without a caching
allocator).  For them the library exports ``mccl_topk_select_noalloc``, whose scratch is a
fixed device array inside the library.  This test loads the shared library with ctypes,
calls the symbol with raw device pointers on two calls in a row (the second call sees the
scratch the first one left behind) and checks both results against the regular entry
point.  It is collected last so that a failure here cannot hide other tests' results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib(native):
    lib = ctypes.CDLL(native.__file__)
    fn = lib.mccl_topk_select_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.mccl_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _k(n, ratio):
    return min(n, max(1, int(n * ratio)))


def test_noalloc_matches_regular_entry_point_twice(native, cuda_device):
    lib = _lib(native)
    stream = torch.cuda.current_stream().cuda_stream
    residual_a = residual_b = None
    for call, (n, ratio, seed) in enumerate([(300_007, 0.01, 1), (70_001, 0.05, 2)]):
        g = torch.randn(n, generator=torch.Generator().manual_seed(seed)).to(cuda_device)
        k = _k(n, ratio)
        # regular entry point (allocates its scratch through torch)
        res_ref = torch.zeros(n, device=cuda_device)
        pairs_ref = native._topk_select(g, res_ref, ratio)
        # allocation-free entry point: every buffer below is the caller's
        res = torch.zeros(n, device=cuda_device)
        pairs = torch.empty(k, 2, dtype=torch.int32, device=cuda_device)
        rc = lib.mccl_topk_select_noalloc(g.data_ptr(), res.data_ptr(), n, k, pairs.data_ptr(), stream)
        assert rc == 0, lib.mccl_noalloc_last_error()
        torch.cuda.synchronize()
        assert pairs_ref.shape == pairs.shape
        assert torch.equal(pairs, pairs_ref), f"call {call}: selected pairs differ"
        assert torch.equal(res, res_ref), f"call {call}: residuals differ"
        # and directly against the host implementation of the same selection rule
        host = native.TopKCompressor(ratio)
        wire = host.compress(g.cpu(), 0)
        import numpy as np
        kk = int(np.frombuffer(wire[:4], dtype=np.uint32)[0])
        rec = np.frombuffer(wire[4:4 + kk * 8], dtype=np.uint32).reshape(kk, 2)
        got = pairs.cpu().numpy().view(np.uint32)
        assert kk == k and np.array_equal(got, rec), f"call {call}: differs from the host compressor"
        assert torch.equal(res.cpu(), host.residual(0)), f"call {call}: residual differs from the host compressor"


def test_noalloc_rejects_bad_sizes(native, cuda_device):
    lib = _lib(native)
    x = torch.zeros(16, device=cuda_device)
    out = torch.empty(16, 2, dtype=torch.int32, device=cuda_device)
    assert lib.mccl_topk_select_noalloc(x.data_ptr(), x.data_ptr(), 16, 0, out.data_ptr(), None) == 1
    assert b"k = 0" in lib.mccl_noalloc_last_error()
    assert lib.mccl_topk_select_noalloc(x.data_ptr(), x.data_ptr(), 16, 17, out.data_ptr(), None) == 1
    assert lib.mccl_topk_select_noalloc(x.data_ptr(), x.data_ptr(), 2**31, 1, out.data_ptr(), None) == 1
    assert b"outside" in lib.mccl_noalloc_last_error()
    assert lib.mccl_topk_select_noalloc(None, x.data_ptr(), 16, 1, out.data_ptr(), None) == 1
