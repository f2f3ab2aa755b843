"""RMSNorm with optional fused residual add and optional output gate.

``rms_norm(x, weight, eps, residual=None, prenorm=False)`` follows the reference module's contract
(fla/modules/layernorm.py:1084-1134): with ``prenorm`` it returns ``(y, residual_out)`` where
``residual_out = x + residual`` is what gets normalised, so a block needs one kernel for "add, then norm".
``rms_norm_gated(x, gate, weight, eps, activation)`` computes ``norm(x) * w * act(gate)`` as
fla/modules/fused_norm_gate.py:992 does for the output of the linear-attention layers.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib

vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
_lib.register("fb_rmsnorm_fwd", [vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, i32, vp])
_lib.register("fb_rmsnorm_bwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, vp])
_lib.register("fb_rmsnorm_bwd_parts", [i64])

_GATE = {None: 0, "swish": 1, "silu": 1, "sigmoid": 2}


def rms_norm_reference(x, weight, eps, residual=None, prenorm=False, gate=None, activation=None):
    r = x if residual is None else x + residual
    rf = r.float()
    y = rf * torch.rsqrt(rf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    if gate is not None:
        g = gate.float()
        y = y * (g * torch.sigmoid(g) if _GATE[activation] == 1 else torch.sigmoid(g))
    y = y.to(x.dtype)
    return (y, r) if prenorm else y


def _kernel_ok(x: torch.Tensor) -> bool:
    return _lib.available() and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, gate, eps, prenorm, gate_mode):
        shape = x.shape
        D = shape[-1]
        x2 = x.reshape(-1, D)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows = x2.shape[0]
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, D)
            res2 = res2 if res2.is_contiguous() else res2.contiguous()
        g2 = None
        if gate is not None:
            g2 = gate.reshape(-1, D)
            g2 = g2 if g2.is_contiguous() else g2.contiguous()
        y = torch.empty_like(x2)
        res_out = torch.empty_like(x2) if (res2 is not None) else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().fb_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(res2), _lib.ptr(weight), _lib.ptr(g2), y.data_ptr(),
                                       _lib.ptr(res_out), rstd.data_ptr(), rows, D, float(eps), gate_mode,
                                       _lib.stream_ptr())
        _lib.check(rc, "fb_rmsnorm_fwd")
        _lib.count_launch()
        xin = res_out if res_out is not None else x2
        ctx.save_for_backward(xin, weight, rstd, g2)
        ctx.shape, ctx.gate_mode, ctx.prenorm, ctx.has_res = shape, gate_mode, prenorm, residual is not None
        ctx.mark_non_differentiable(rstd)
        if prenorm:
            return y.view(shape), (res_out if res_out is not None else x2).view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy, dres_out=None):
        xin, weight, rstd, g2 = ctx.saved_tensors
        D = ctx.shape[-1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, D)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres2 = None
        if ctx.prenorm and dres_out is not None:
            dres2 = dres_out.reshape(-1, D)
            dres2 = dres2 if dres2.is_contiguous() else dres2.contiguous()
        L = _lib.lib()
        dx = torch.empty_like(xin)
        dgate = torch.empty_like(xin) if g2 is not None else None
        dw = None
        dw_part = None
        if weight is not None:
            parts = int(L.fb_rmsnorm_bwd_parts(rows))
            dw_part = torch.empty(parts, D, dtype=torch.float32, device=xin.device)
            mg = getattr(weight, "main_grad", None)
            dw = mg if mg is not None else torch.empty(D, dtype=torch.float32, device=xin.device)
        rc = L.fb_rmsnorm_bwd(dy2.data_ptr(), xin.data_ptr(), _lib.ptr(weight), rstd.data_ptr(), _lib.ptr(g2),
                              _lib.ptr(dres2), dx.data_ptr(), _lib.ptr(dgate), _lib.ptr(dw_part), _lib.ptr(dw), rows, D,
                              ctx.gate_mode, 1 if (weight is not None and hasattr(weight, "main_grad")) else 0,
                              _lib.stream_ptr())
        _lib.check(rc, "fb_rmsnorm_bwd")
        _lib.count_launch(2 if weight is not None else 1)
        dxv = dx.view(ctx.shape)
        gw = None
        if weight is not None and not hasattr(weight, "main_grad"):
            gw = dw.to(weight.dtype)
        gres = dxv if ctx.has_res else None
        ggate = dgate.view(ctx.shape) if dgate is not None else None
        return dxv, gw, gres, ggate, None, None, None


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6,
             residual: Optional[torch.Tensor] = None, prenorm: bool = False):
    if _kernel_ok(x):
        return _RMSNormFn.apply(x, weight, residual, None, eps, prenorm, 0)
    return rms_norm_reference(x, weight, eps, residual, prenorm)


def rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6,
                   activation: str = "swish"):
    if _kernel_ok(x):
        return _RMSNormFn.apply(x, weight, None, gate, eps, False, _GATE[activation])
    return rms_norm_reference(x, weight, eps, gate=gate, activation=activation)
