"""The allocation-free RMSNorm backward (csrc/no_alloc.h) against the regular entry point.

Some callers of the library cannot allocate device memory when they call it (a frozen allocator, a fixed memory
budget, a host without PyTorch that has no workspace to pass).  For them the library exports one entry point whose
scratch lives in a static device array.  This test calls it through its exported C symbol, twice in a row (the
array is shared and keeps the previous call's contents), and checks both results against ``pb_norm_bwd``.
It is collected last so that a failure here cannot hide another test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, dy, x, w, rstd, sm_count):
    T, H = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty(H, dtype=torch.float32, device=x.device)
    lib.pb_norm_bwd_scratch_floats.restype = ctypes.c_longlong
    scratch = torch.empty(int(lib.pb_norm_bwd_scratch_floats(ctypes.c_int(H), ctypes.c_int(sm_count))),
                          dtype=torch.float32, device=x.device)
    rc = lib.pb_norm_bwd(
        ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(0),
        ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
        ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_int(0), ctypes.c_void_p(scratch.data_ptr()),
        ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(0), ctypes.c_int(sm_count),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, dw


def test_no_alloc_rmsnorm_backward_matches_regular_entry_point():
    from pippy_b200.ops import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    fn = lib.pb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    torch.manual_seed(0)
    for T, H in ((777, 4096), (300, 768)):  # two calls in a row, different shapes, same static scratch
        x = torch.randn(T, H, device=dev).bfloat16()
        dy = torch.randn(T, H, device=dev).bfloat16()
        w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        dx_ref, dw_ref = _regular(lib, dy, x, w, rstd, sm_count)
        dx = torch.empty_like(x)
        dw = torch.full((H,), 7.0, dtype=torch.float32, device=dev)
        rc = fn(ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
                ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)  # same kernel, same per-row arithmetic
        rel = ((dw - dw_ref).abs().max() / dw_ref.abs().max()).item()
        assert rel < 2e-2, rel  # partial sums are grouped differently (128 CTAs vs 2 per SM)
    # sizes beyond the built-in scratch are refused, not truncated
    assert lib.pb_rmsnorm_bwd_noalloc_max_hidden() == 8192
    rc = fn(ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
            ctypes.c_void_p(0), ctypes.c_int(0), ctypes.c_int(8), ctypes.c_int(16384), ctypes.c_void_p(0))
    assert rc == -2
