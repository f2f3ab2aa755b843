"""Flat-buffer optimizer kernels: sum of squares (gradient norm) and AdamW with clipping and skip-on-NaN.

All control values live on the device (``ctrl``: ``[norm_sq, step, skipped, clip_coef, norm]``), so a training
step needs no host synchronisation: the clip coefficient and the "skip this step if the norm is NaN/Inf"
decision (flame/train.py:518-525 makes it on the host every step) are taken inside the kernels.
Update rule = ``torch.optim.AdamW``.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib

vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
_lib.register("fb_sumsq", [vp, i64, vp, vp, i32, vp])
_lib.register("fb_sumsq_parts", [])
_lib.register("fb_adamw", [vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, i32, vp, f32, vp])
_lib.register("fb_adamw_finalize", [vp, f32, i32, f32, vp])
_lib.register("fb_cast_f32_bf16", [vp, vp, i64, vp])
_lib.register("fb_status_to_ctrl", [vp, vp])

CTRL_NORM_SQ, CTRL_STEP, CTRL_SKIPPED, CTRL_COEF, CTRL_NORM, CTRL_ABORT, CTRL_ABORTED = 0, 1, 2, 3, 4, 5, 6
CTRL_SIZE = 8


def latch_status(ctrl: torch.Tensor) -> None:
    """Copies "the library status word is non-zero" into ``ctrl[CTRL_ABORT]`` on the stream, so that the update kernels
    launched after it apply nothing when a bounded wait (a peer flag, a pipeline barrier) ran out earlier in the step:
    half-reduced gradients never reach the parameters.  The host learns of it from ``_lib.status()`` without a sync."""
    if _kernel_ok(ctrl):
        _lib.check(_lib.lib().fb_status_to_ctrl(ctrl.data_ptr(), _lib.stream_ptr()), "fb_status_to_ctrl")
        _lib.count_launch()


def _kernel_ok(t: torch.Tensor) -> bool:
    return _lib.available() and t.is_cuda and t.dtype == torch.float32


def sumsq_accumulate(x: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None,
                     accumulate: bool = True) -> None:
    """``out[0] (+)= sum(x*x)`` for a flat fp32 tensor, reduced in a fixed order."""
    if _kernel_ok(x):
        L = _lib.lib()
        if scratch is None or scratch.numel() < L.fb_sumsq_parts():
            scratch = torch.empty(int(L.fb_sumsq_parts()), dtype=torch.float32, device=x.device)
        rc = L.fb_sumsq(x.data_ptr(), x.numel(), scratch.data_ptr(), out.data_ptr(), 1 if accumulate else 0,
                        _lib.stream_ptr())
        _lib.check(rc, "fb_sumsq")
        _lib.count_launch(2)
    else:
        s = x.float().pow(2).sum()
        if accumulate:
            out[0] += s
        else:
            out[0] = s


def adamw_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, p_lowp: Optional[torch.Tensor],
               ctrl: torch.Tensor, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
               max_norm: float, skip_nan_inf: bool, grad_scale: float = 1.0) -> None:
    """One AdamW update of a flat fp32 shard; ``ctrl[0]`` must hold the global gradient norm squared.  A negative
    ``weight_decay`` selects plain Adam with L2 decay ``|weight_decay|`` (see ``OptimConfig.kernel_weight_decay``)."""
    if _kernel_ok(p):
        rc = _lib.lib().fb_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _lib.ptr(p_lowp), p.numel(),
                                 lr, beta1, beta2, eps, weight_decay, max_norm, 1 if skip_nan_inf else 0,
                                 ctrl.data_ptr(), grad_scale, _lib.stream_ptr())
        _lib.check(rc, "fb_adamw")
        _lib.count_launch()
        return
    if float(ctrl[CTRL_ABORT]) != 0.0:
        return
    norm = math.sqrt(float(ctrl[CTRL_NORM_SQ])) * grad_scale if not math.isnan(float(ctrl[CTRL_NORM_SQ])) else float("nan")
    if skip_nan_inf and not math.isfinite(norm):
        return
    coef = min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0
    coef *= grad_scale
    step = float(ctrl[CTRL_STEP]) + 1.0
    gr = g * coef
    if weight_decay < 0:  # plain Adam: the decay enters through the gradient (``torch.optim.Adam(weight_decay=...)``)
        gr = gr + (-weight_decay) * p
        weight_decay = 0.0
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gr, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gr, gr, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if p_lowp is not None:
        p_lowp.copy_(p)


def adamw_finalize(ctrl: torch.Tensor, max_norm: float, skip_nan_inf: bool, grad_scale: float = 1.0) -> None:
    """Advance the device-side counters once all shards of this step were updated."""
    if _kernel_ok(ctrl):
        rc = _lib.lib().fb_adamw_finalize(ctrl.data_ptr(), max_norm, 1 if skip_nan_inf else 0, grad_scale,
                                          _lib.stream_ptr())
        _lib.check(rc, "fb_adamw_finalize")
        _lib.count_launch()
        return
    nsq = float(ctrl[CTRL_NORM_SQ])
    norm = math.sqrt(nsq) * grad_scale if nsq == nsq and nsq >= 0 else float("nan")
    if float(ctrl[CTRL_ABORT]) != 0.0:
        ctrl[CTRL_ABORTED] += 1
        ctrl[CTRL_COEF] = 0
    elif skip_nan_inf and not math.isfinite(norm):
        ctrl[CTRL_SKIPPED] += 1
        ctrl[CTRL_COEF] = 0
    else:
        ctrl[CTRL_STEP] += 1
        ctrl[CTRL_COEF] = min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0
    ctrl[CTRL_NORM] = norm


def cast_to_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    if _kernel_ok(src) and dst.dtype == torch.bfloat16:
        rc = _lib.lib().fb_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.stream_ptr())
        _lib.check(rc, "fb_cast_f32_bf16")
        _lib.count_launch()
    else:
        dst.copy_(src)
