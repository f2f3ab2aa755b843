"""Depthwise causal short convolution over packed sequences (``csrc/conv.cu``).

``short_conv(x, weight, bias, meta, activation)``: x ``[T, D]``, weight ``[D, 1, W]`` (the layout of
``nn.Conv1d(D, D, W, groups=D)``), optional SiLU.  Replaces the Triton kernels behind
``fla.modules.ShortConvolution`` (fla/modules/conv/triton/kernels.py:37-345).
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib, linear_attn as la
from .varlen import VarlenMeta

vp, i32, i64 = c_void_p, c_int, c_longlong
_lib.register("fb_short_conv_strips", [i64])
_lib.register("fb_short_conv_fwd", [vp, vp, vp, vp, vp, i64, i32, i32, i64, i64, i32, vp])
_lib.register("fb_short_conv_bwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i64, i64, i32, i32, vp])


class _ShortConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, meta: VarlenMeta, silu: bool):
        T, D = x.shape
        W = weight.shape[-1]
        x = x if (x.stride(1) == 1 and x.stride(0) % 8 == 0) else x.contiguous()
        w2 = weight.reshape(D, W)
        y = torch.empty(T, D, dtype=x.dtype, device=x.device)
        pos = meta.position_ids
        rc = _lib.lib().fb_short_conv_fwd(x.data_ptr(), w2.data_ptr(), _lib.ptr(bias), pos.data_ptr(), y.data_ptr(), T, D,
                                          W, x.stride(0), y.stride(0), 1 if silu else 0, _lib.stream_ptr())
        _lib.check(rc, "fb_short_conv_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x, weight, bias)
        ctx.meta, ctx.silu = meta, silu
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        T, D = x.shape
        W = weight.shape[-1]
        L = _lib.lib()
        dy = dy if dy.is_contiguous() else dy.contiguous()
        w2 = weight.reshape(D, W)
        dx = torch.empty(T, D, dtype=x.dtype, device=x.device)
        dpre = torch.empty(T, D, dtype=x.dtype, device=x.device)
        strips = int(L.fb_short_conv_strips(T))
        part = torch.empty(strips, D, W + 1, dtype=torch.float32, device=x.device)
        mg_w = getattr(weight, "main_grad", None)
        mg_b = getattr(bias, "main_grad", None) if bias is not None else None
        use_main = mg_w is not None and (bias is None or mg_b is not None)
        dw = mg_w.view(D, W) if use_main else torch.empty(D, W, dtype=torch.float32, device=x.device)
        db = None
        if bias is not None:
            db = mg_b if use_main else torch.empty(D, dtype=torch.float32, device=x.device)
        # dx is written with the row stride of x only when x is contiguous; keep both contiguous
        xs = x if x.is_contiguous() else x.contiguous()
        rc = L.fb_short_conv_bwd(dy.data_ptr(), xs.data_ptr(), w2.data_ptr(), _lib.ptr(bias), ctx.meta.position_ids.data_ptr(),
                                 dx.data_ptr(), dpre.data_ptr(), part.data_ptr(), dw.data_ptr(), _lib.ptr(db), T, D, W,
                                 xs.stride(0), dy.stride(0), 1 if ctx.silu else 0, 1 if use_main else 0, _lib.stream_ptr())
        _lib.check(rc, "fb_short_conv_bwd")
        _lib.count_launch(3)
        gw = None if use_main else dw.view_as(weight).to(weight.dtype)
        gb = None if (bias is None or use_main) else db.to(bias.dtype)
        return dx, gw, gb, None, None


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], meta: VarlenMeta,
               activation: Optional[str] = "silu") -> torch.Tensor:
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None and weight.shape[-1] > 1:
        return _short_conv_with_halo(x, weight, bias, meta, activation, sl)
    if (_lib.available() and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and weight.shape[-1] <= 8):
        return _ShortConvFn.apply(x, weight, bias, meta, activation in ("silu", "swish"))
    return la.short_conv(x, weight, bias, meta, activation)



class _PositionsOnly:
    """The part of a ``VarlenMeta`` the convolution reads."""

    def __init__(self, position_ids: torch.Tensor) -> None:
        self.position_ids = position_ids


def _short_conv_with_halo(x, weight, bias, meta, activation, sl) -> torch.Tensor:
    """The convolution on one rank's slice of a row that context parallelism cut inside documents: the ``W - 1`` rows
    in front of the slice come from the previous rank (every rank contributes its last ``W - 1`` rows to one
    differentiable all-gather), are put in front of the local rows with the document positions they have, and their
    outputs are dropped.  ``meta.position_ids`` count from the start of the whole document, so the taps' own validity
    rule (a tap reaches back at most ``position`` rows) also decides what the halo may contribute.  Counterpart of fla's
    convolution tail exchange, also an all-gather followed by an index (fla/ops/cp/comm.py:64-169)."""
    from ..parallel.context_parallel import _AllGatherRows
    h = weight.shape[-1] - 1
    assert x.shape[0] >= h, "a context-parallel slice shorter than the convolution"
    tails = _AllGatherRows.apply(x[-h:].contiguous(), sl.group)          # [world * h, D]
    if sl.rank > 0 and sl.continues[sl.rank]:
        halo = tails[(sl.rank - 1) * h: sl.rank * h]
    else:
        halo = torch.zeros(h, x.shape[1], dtype=x.dtype, device=x.device)
    pos = meta.position_ids
    front = pos[:1] - h + torch.arange(h, device=pos.device, dtype=pos.dtype)   # negative: rows of an earlier document
    ext = _PositionsOnly(torch.cat([front, pos]).contiguous())
    y = short_conv(torch.cat([halo, x], 0), weight, bias, ext, activation)[h:]
    # every rank takes part in the gather's backward collective, also one that uses nobody's rows
    return y + tails[:0].sum().to(y.dtype)   # an empty slice: connected to the gather, independent of its values
