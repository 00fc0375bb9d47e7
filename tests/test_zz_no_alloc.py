"""The allocation-free C entry point `nfb200_linear_add_noalloc`, called through its exported symbol.

Some hosts of this library cannot allocate device memory when they call it: a plugin that only receives
raw device pointers from a foreign runtime, or a process whose memory was handed over up front.  For them the
library offers one entry point whose split-K scratch is a static device array inside the library.  This test
calls it with ctypes (no torch binding in between), twice in a row because every call reuses the same
scratch, and compares both results with the library's ordinary `linear + residual add` path.  It must hold
when run on its own and when run last after every other GPU test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ninfer_fusion_b200", "_C.so")


def _entry():
    import ninfer_fusion_b200

    ninfer_fusion_b200.load_native()       # torch's own libraries must be loaded before the shared object
    lib = ctypes.CDLL(LIB)
    fn = lib.nfb200_linear_add_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_int]
    return fn


def _call(fn, x, w, resid, splits):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), resid.data_ptr(), x.shape[0], w.shape[0],
            x.shape[1], splits, ctypes.c_void_p(stream), err, 256)
    return rc, err.value.decode()


def test_no_alloc_linear_add_matches_regular_path_twice(ops):
    fn = _entry()
    torch.manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # set-up call: looks up the scratch array's address; with lazy module loading this is also the moment the
    # driver instantiates the library's static 16 MiB array, so device memory may shrink here and only here
    x0 = torch.zeros(1, 64, device="cuda", dtype=torch.bfloat16)
    w0 = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, x0, w0, torch.zeros(1, 8, device="cuda", dtype=torch.bfloat16), 1)
    torch.cuda.synchronize()
    assert rc == 0, msg
    for T, N, K, splits in [(32, 5120, 6144, 0), (7, 640, 2560, 4)]:   # second call reuses (dirty) scratch
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        resid = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        # existing entry point: tcgen05 GEMM with the residual epilogue
        expect = resid.clone()
        ops.gemm_bf16(x, w, expect, 1, expect, None, None, 1, status, False)
        got = resid.clone()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()     # the driver's own count: sees allocations torch does not make
        rc, msg = _call(fn, x, w, got, splits)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == before
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, f"device memory shrank by {free_before - free_after} bytes during the call"
        ref = resid.float() + x.float() @ w.float().t()
        scale = ref.abs().max().item()
        assert (got.float() - expect.float()).abs().max().item() / scale < 2e-2
        assert (got.float() - ref).abs().max().item() / scale < 2e-2
    assert int(status.item()) == 0


def test_no_alloc_refuses_oversized_and_bad_arguments():
    fn = _entry()
    x = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(8192, 64, device="cuda", dtype=torch.bfloat16)
    resid = torch.zeros(256, 8192, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, x, w, resid, 8)          # 8 * 256 * 8192 floats > 4 Mi
    assert rc == 2 and "exceeds the built-in scratch" in msg
    rc, msg = _call(fn, x[:0], w, resid, 1)
    assert rc == 1
    big_t = torch.zeros(300, 64, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, big_t, w, resid, 1)
    assert rc == 2 and "T must be" in msg
    # limits of the residual update are checked on the host, before anything is launched
    x8 = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    wide_w = torch.zeros(8200, 64, device="cuda", dtype=torch.bfloat16)
    wide_r = torch.full((8, 8200), 3.0, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, x8, wide_w, wide_r, 1)
    assert rc == 2 and "N must be <= 8192" in msg
    odd_w = torch.zeros(36, 64, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, x8, odd_w, torch.zeros(8, 36, device="cuda", dtype=torch.bfloat16), 1)
    assert rc == 1 and "multiple of 8" in msg
    w64 = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    backing = torch.full((8 * 64 + 8,), 3.0, device="cuda", dtype=torch.bfloat16)
    misaligned = backing[1:1 + 8 * 64].view(8, 64)          # 2 bytes past a 16-byte boundary
    rc, msg = _call(fn, x8, w64, misaligned, 1)
    assert rc == 1 and "16-byte aligned" in msg
    torch.cuda.synchronize()
    assert bool((wide_r == 3.0).all()) and bool((backing == 3.0).all())   # a refused call touches nothing
