"""Fused gate arithmetic of the linear-attention layers (one kernel pass each way instead of a chain of elementwise
framework kernels).

``hgrn2_gates(q_raw, f_raw, lower_bound)`` returns ``(q, k, g)`` of fla/layers/hgrn2.py:160-190:
``q = silu(q_raw)``, ``g = logsigmoid(f_raw)`` (with a lower bound: ``g = log(lb + (1 - lb) sigmoid(f_raw))``, the closed
form of the reference's ``logaddexp(log lb, log1p(-lb) + logsigmoid f)``), ``k = 1 - exp(g)``; ``g`` in fp32.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

_lib.register("fb_hgrn2_gate_tiles", [c_longlong])
_lib.register("fb_hgrn2_gate_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
_lib.register("fb_hgrn2_gate_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_longlong, c_int, c_void_p])


def hgrn2_gates_reference(q_raw: torch.Tensor, f_raw: torch.Tensor,
                          lower_bound: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    q = F.silu(q_raw)
    g = F.logsigmoid(f_raw.float())
    if lower_bound is not None:
        lb = lower_bound.float()
        g = torch.logaddexp(lb.log(), torch.log1p(-lb) + g)
    k = (1 - g.exp()).to(q_raw.dtype)
    return q, k, g


class _Hgrn2Gates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_raw, f_raw, lb):
        rows, D = q_raw.shape
        q_raw, f_raw = q_raw.contiguous(), f_raw.contiguous()
        lbf = lb.detach().float().contiguous() if lb is not None else None
        q, k = torch.empty_like(q_raw), torch.empty_like(q_raw)
        g = torch.empty(rows, D, dtype=torch.float32, device=q_raw.device)
        rc = _lib.lib().fb_hgrn2_gate_fwd(q_raw.data_ptr(), f_raw.data_ptr(), _lib.ptr(lbf), q.data_ptr(), k.data_ptr(),
                                          g.data_ptr(), rows, D, _lib.stream_ptr())
        _lib.check(rc, "fb_hgrn2_gate_fwd")
        _lib.count_launch()
        ctx.save_for_backward(q_raw, f_raw, lbf)
        ctx.lb_dtype = lb.dtype if lb is not None else None
        return q, k, g

    @staticmethod
    def backward(ctx, dq, dk, dg):
        q_raw, f_raw, lbf = ctx.saved_tensors
        rows, D = q_raw.shape
        L = _lib.lib()
        dq = torch.zeros_like(q_raw) if dq is None else dq.contiguous()
        dk = torch.zeros_like(q_raw) if dk is None else dk.contiguous()
        dg = torch.zeros(rows, D, dtype=torch.float32, device=q_raw.device) if dg is None else dg.float().contiguous()
        dq_raw, df_raw = torch.empty_like(q_raw), torch.empty_like(f_raw)
        part = dlb = None
        if lbf is not None:
            part = torch.empty(int(L.fb_hgrn2_gate_tiles(rows)), D, dtype=torch.float32, device=q_raw.device)
            dlb = torch.empty(D, dtype=torch.float32, device=q_raw.device)
        rc = L.fb_hgrn2_gate_bwd(q_raw.data_ptr(), f_raw.data_ptr(), _lib.ptr(lbf), dq.data_ptr(), dk.data_ptr(), dg.data_ptr(),
                                 dq_raw.data_ptr(), df_raw.data_ptr(), _lib.ptr(part), _lib.ptr(dlb), rows, D, _lib.stream_ptr())
        _lib.check(rc, "fb_hgrn2_gate_bwd")
        _lib.count_launch(2 if lbf is not None else 1)
        return dq_raw, df_raw, (dlb.to(ctx.lb_dtype) if dlb is not None else None)


def hgrn2_gates(q_raw: torch.Tensor, f_raw: torch.Tensor,
                lower_bound: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[T, D]`` bf16 projections (and an optional ``[D]`` lower bound) -> ``q`` bf16, ``k`` bf16, ``g`` fp32, all ``[T, D]``."""
    if (_lib.available() and q_raw.is_cuda and q_raw.dtype == torch.bfloat16 and f_raw.dtype == torch.bfloat16
            and q_raw.dim() == 2 and q_raw.shape == f_raw.shape and q_raw.shape[1] % 8 == 0):
        return _Hgrn2Gates.apply(q_raw, f_raw, lower_bound)
    return hgrn2_gates_reference(q_raw, f_raw, lower_bound)


# ----------------------------------------------------------------------------------------------------------------------
# Mamba2: the elementwise work around the SSD core (fla/layers/mamba2.py:241-331)
# ----------------------------------------------------------------------------------------------------------------------
_lib.register("fb_mamba2_pre_fwd", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_longlong, c_int, c_int, c_void_p])
_lib.register("fb_mamba2_pre_bwd", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p])
_lib.register("fb_mamba2_post_fwd", [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int,
                                     c_int, c_void_p])
_lib.register("fb_mamba2_post_bwd", [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p])


class SplitColumns(torch.autograd.Function):
    """Column blocks of a ``[T, N]`` matrix as views; the backward writes the blocks' gradients side by side in ONE pass
    (autograd's own slice backward zero-fills a full-width matrix per block and adds them up)."""

    @staticmethod
    def forward(ctx, x, *sizes):
        ctx.sizes, ctx.dtype = sizes, x.dtype
        outs, c = [], 0
        for n in sizes:
            outs.append(x[:, c:c + n])
            c += n
        assert c == x.shape[1], (sizes, x.shape)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        T = next(g.shape[0] for g in grads if g is not None)
        dev = next(g.device for g in grads if g is not None)
        parts = [g.to(ctx.dtype) if g is not None else torch.zeros(T, n, dtype=ctx.dtype, device=dev)
                 for g, n in zip(grads, ctx.sizes)]
        return (torch.cat(parts, dim=1), *([None] * len(ctx.sizes)))


def split_columns(x: torch.Tensor, sizes) -> Tuple[torch.Tensor, ...]:
    return SplitColumns.apply(x, *sizes)


def _views_ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
               and t.data_ptr() % 16 == 0 for t in ts)


class _Mamba2Pre(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt_raw, dt_bias, A_log, H, P):
        T = x.shape[0]
        bias32, alog32 = dt_bias.detach().float().contiguous(), A_log.detach().float().contiguous()
        xv = torch.empty(T, H, P, dtype=x.dtype, device=x.device)
        dt = torch.empty(T, H, dtype=torch.float32, device=x.device)
        g = torch.empty(T, H, dtype=torch.float32, device=x.device)
        rc = _lib.lib().fb_mamba2_pre_fwd(x.data_ptr(), x.stride(0), dt_raw.data_ptr(), dt_raw.stride(0), bias32.data_ptr(),
                                          alog32.data_ptr(), xv.data_ptr(), dt.data_ptr(), g.data_ptr(), T, H, P,
                                          _lib.stream_ptr())
        _lib.check(rc, "fb_mamba2_pre_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x, dt_raw, bias32, alog32, dt)
        ctx.dims = (H, P)
        ctx.dtypes = (dt_bias.dtype, A_log.dtype, dt_raw.dtype)
        return xv, dt, g

    @staticmethod
    def backward(ctx, dxv, ddt, dg):
        x, dt_raw, bias32, alog32, dt = ctx.saved_tensors
        H, P = ctx.dims
        T = x.shape[0]
        dxv = torch.zeros(T, H, P, dtype=x.dtype, device=x.device) if dxv is None else dxv.contiguous()
        dg = torch.zeros(T, H, dtype=torch.float32, device=x.device) if dg is None else dg.float().contiguous()
        ddt = None if ddt is None else ddt.float().contiguous()
        dx = torch.empty(T, H * P, dtype=x.dtype, device=x.device)
        d_raw = torch.empty(T, H, dtype=torch.float32, device=x.device)
        rc = _lib.lib().fb_mamba2_pre_bwd(x.data_ptr(), x.stride(0), dt_raw.data_ptr(), dt_raw.stride(0), bias32.data_ptr(),
                                          alog32.data_ptr(), dxv.data_ptr(), dg.data_ptr(), _lib.ptr(ddt), dx.data_ptr(),
                                          d_raw.data_ptr(), T, H, P, _lib.stream_ptr())
        _lib.check(rc, "fb_mamba2_pre_bwd")
        _lib.count_launch()
        d_bias = d_raw.sum(0)
        d_alog = (dg * dt).sum(0) * (-alog32.exp())     # g = A dt with A = -exp(A_log): dA_log = dA * A
        return (dx, d_raw.to(ctx.dtypes[2]), d_bias.to(ctx.dtypes[0]), d_alog.to(ctx.dtypes[1]), None, None)


class _Mamba2Post(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, x, z, D, H, P):
        T = x.shape[0]
        y = y.contiguous()
        d32 = D.detach().float().contiguous()
        out = torch.empty(T, H * P, dtype=x.dtype, device=x.device)
        rc = _lib.lib().fb_mamba2_post_fwd(y.data_ptr(), x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0), d32.data_ptr(),
                                           out.data_ptr(), T, H, P, _lib.stream_ptr())
        _lib.check(rc, "fb_mamba2_post_fwd")
        _lib.count_launch()
        ctx.save_for_backward(y, x, z, d32)
        ctx.dims, ctx.d_dtype = (H, P), D.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        y, x, z, d32 = ctx.saved_tensors
        H, P = ctx.dims
        T = x.shape[0]
        dout = dout.contiguous()
        dy = torch.empty(T, H, P, dtype=x.dtype, device=x.device)
        dx = torch.empty(T, H * P, dtype=x.dtype, device=x.device)
        dz = torch.empty(T, H * P, dtype=x.dtype, device=x.device)
        part = torch.empty(T, H, dtype=torch.float32, device=x.device)
        rc = _lib.lib().fb_mamba2_post_bwd(y.data_ptr(), x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0), d32.data_ptr(),
                                           dout.data_ptr(), dy.data_ptr(), dx.data_ptr(), dz.data_ptr(), part.data_ptr(), T, H, P,
                                           _lib.stream_ptr())
        _lib.check(rc, "fb_mamba2_post_bwd")
        _lib.count_launch()
        return dy, dx, dz, part.sum(0).to(ctx.d_dtype), None, None


def mamba2_pre_reference(x, dt_raw, dt_bias, A_log, H: int, P: int):
    T = x.shape[0]
    dt = F.softplus(dt_raw.float() + dt_bias.float())
    g = dt * (-torch.exp(A_log.float()))[None, :]
    xv = (x.reshape(T, H, P).float() * dt[..., None]).to(x.dtype)
    return xv, dt, g


def mamba2_post_reference(y, x, z, D, H: int, P: int):
    T = x.shape[0]
    u = y.reshape(T, H, P).float() + x.reshape(T, H, P).float() * D.float()[None, :, None]
    return (u.reshape(T, H * P) * F.silu(z.float())).to(x.dtype)


def mamba2_pre(x, dt_raw, dt_bias, A_log, H: int, P: int):
    """``x [T, H * P]`` and ``dt_raw [T, H]`` (strided views are fine) -> ``xv = x dt`` ``[T, H, P]``, ``dt = softplus(dt_raw +
    dt_bias)`` and the log decay ``g = -exp(A_log) dt`` (both fp32 ``[T, H]``), in one kernel."""
    if _lib.available() and P in (64, 128, 256) and _views_ok(x) and dt_raw.is_cuda and dt_raw.dtype == torch.bfloat16 \
            and dt_raw.stride(1) == 1:
        return _Mamba2Pre.apply(x, dt_raw, dt_bias, A_log, H, P)
    return mamba2_pre_reference(x, dt_raw, dt_bias, A_log, H, P)


def mamba2_post(y, x, z, D, H: int, P: int):
    """``(y + D x) silu(z)`` as ``[T, H * P]`` in one kernel; ``x`` and ``z`` may be strided views."""
    if _lib.available() and P in (64, 128, 256) and _views_ok(x, z) and y.is_cuda and y.dtype == torch.bfloat16:
        return _Mamba2Post.apply(y, x, z, D, H, P)
    return mamba2_post_reference(y, x, z, D, H, P)
