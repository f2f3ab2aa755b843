"""The allocation-free RMSNorm backward, called through its exported C symbol, against the regular entry point.

Some users of the kernel library cannot allocate device memory when they need a result (they run inside another
framework's memory pool, or in a loop that must stay clear of the driver's allocator).  For them the library exports
``fb_rmsnorm_bwd_noalloc``, whose scratch is a fixed array inside the library image.  This test drives that symbol with
raw pointers, twice in a row (the scratch is shared between calls), and checks both results against
``fb_rmsnorm_bwd`` given caller-allocated scratch, and the size limit against its documented maximum.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_noalloc_rmsnorm_backward_matches_regular_entry_point():
    from flame_b200.ops import _build, _lib
    lib = ctypes.CDLL(str(_build.LIB_PATH))  # the exported C symbols, nothing else
    noalloc = lib.fb_rmsnorm_bwd_noalloc
    noalloc.restype = ctypes.c_int
    noalloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    regular = lib.fb_rmsnorm_bwd
    regular.restype = ctypes.c_int
    regular.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    parts_fn = lib.fb_rmsnorm_bwd_parts
    parts_fn.restype = ctypes.c_int
    parts_fn.argtypes = [ctypes.c_longlong]

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(0)
    for call, (rows, D) in enumerate([(3001, 1024), (517, 2304)]):
        x = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(D, device=dev)).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
        # regular entry point with caller-provided scratch
        dx_ref = torch.empty_like(x)
        dw_ref = torch.zeros(D, device=dev)
        scratch = torch.empty(parts_fn(rows), D, device=dev)
        rc = regular(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), None, None, _ptr(dx_ref), None, _ptr(scratch), _ptr(dw_ref),
                     rows, D, 0, 0, stream)
        assert rc == 0
        # allocation-free entry point: inputs and outputs only
        dx = torch.empty_like(x)
        dw = torch.zeros(D, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        rc = noalloc(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(dw), rows, D, 0, stream)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert torch.equal(dx, dx_ref)
        assert torch.allclose(dw, dw_ref, rtol=1e-5, atol=1e-5)
        # and against the definition, within the tolerance of the other kernel tests
        xf, wf, dyf = x.float().requires_grad_(True), w.float().requires_grad_(True), dy.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
        y.backward(dyf)
        err = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
        assert err(dx, xf.grad) < 2e-2 and err(dw, wf.grad) < 2e-2
    # sizes beyond the documented maximum are refused, not truncated
    big = 4096 + 8
    t = torch.zeros(8, big, device=dev, dtype=torch.bfloat16)
    rc = noalloc(_ptr(t), _ptr(t), _ptr(t[0]), _ptr(torch.ones(8, device=dev)), _ptr(torch.empty_like(t)),
                 _ptr(torch.zeros(big, device=dev)), 8, big, 0, stream)
    assert rc != 0
    _lib.assert_status_ok()
