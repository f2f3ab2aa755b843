"""SwiGLU on a fused ``[T, 2I]`` gate/up buffer: ``a = silu(gate) * up``.

The backward writes ``d_gate`` and ``d_up`` side by side into one ``[T, 2I]`` buffer so the weight gradient
of the fused gate/up projection is a single GEMM.  Same math as fla/modules/activations.py:553-628.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p

import torch
import torch.nn.functional as F

from . import _lib

vp, i32, i64 = c_void_p, c_int, c_longlong
_lib.register("fb_swiglu_fwd", [vp, vp, vp, i64, i32, i64, i64, i64, vp])
_lib.register("fb_swiglu_bwd", [vp, vp, vp, vp, vp, vp, i64, i32, i64, i64, i64, i64, i64, i64, vp])


def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shape = gu.shape
        I = shape[-1] // 2
        gu2 = gu.reshape(-1, 2 * I)
        gu2 = gu2 if gu2.is_contiguous() else gu2.contiguous()
        T = gu2.shape[0]
        a = torch.empty(T, I, dtype=gu.dtype, device=gu.device)
        rc = _lib.lib().fb_swiglu_fwd(gu2.data_ptr(), gu2.data_ptr() + 2 * I, a.data_ptr(), T, I, 2 * I, 2 * I, I,
                                      _lib.stream_ptr())
        _lib.check(rc, "fb_swiglu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(gu2)
        ctx.shape = shape
        return a.view(*shape[:-1], I)

    @staticmethod
    def backward(ctx, da):
        (gu2,) = ctx.saved_tensors
        T, I2 = gu2.shape
        I = I2 // 2
        da2 = da.reshape(-1, I)
        da2 = da2 if da2.is_contiguous() else da2.contiguous()
        dgu = torch.empty_like(gu2)
        rc = _lib.lib().fb_swiglu_bwd(da2.data_ptr(), gu2.data_ptr(), gu2.data_ptr() + 2 * I, dgu.data_ptr(),
                                      dgu.data_ptr() + 2 * I, 0, T, I, I, I2, I2, I2, I2, I, _lib.stream_ptr())
        _lib.check(rc, "fb_swiglu_bwd")
        _lib.count_launch()
        return dgu.view(ctx.shape)


def swiglu_backward(da2: torch.Tensor, gu2: torch.Tensor) -> torch.Tensor:
    """``[d_gate | d_up]`` for ``a = silu(gate) * up`` from ``da [T, I]`` and the saved ``[gate | up] [T, 2 I]``."""
    T, I2 = gu2.shape
    I = I2 // 2
    dgu = torch.empty_like(gu2)
    rc = _lib.lib().fb_swiglu_bwd(da2.data_ptr(), gu2.data_ptr(), gu2.data_ptr() + 2 * I, dgu.data_ptr(),
                                  dgu.data_ptr() + 2 * I, 0, T, I, I, I2, I2, I2, I2, I, _lib.stream_ptr())
    _lib.check(rc, "fb_swiglu_bwd")
    _lib.count_launch()
    return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    if _lib.available() and gu.is_cuda and gu.dtype == torch.bfloat16 and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLUFn.apply(gu)
    return swiglu_reference(gu)
