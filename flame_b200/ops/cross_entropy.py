"""Cross-entropy heads.

``fused_linear_cross_entropy(x, weight, labels)`` never materialises the full ``[T, V]`` logits: tokens are
processed in chunks; per chunk one tcgen05 GEMM produces bf16 logits, one kernel turns them into
``softmax - onehot`` in place (and emits the per-row loss), and two more GEMMs turn that into ``dx`` and the
weight gradient.  Gradients are therefore produced during the forward, as in
fla/modules/fused_linear_cross_entropy.py:274-407, but the number of valid targets stays on the device
(that file syncs the host with ``.item()`` at line 322).

``cross_entropy(logits, labels)`` is the plain row-wise loss with in-place gradient
(fla/modules/fused_cross_entropy.py:31-156).  Labels equal to ``ignore_index`` contribute nothing.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import gemm_nn, gemm_nt, gemm_tn

vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
_lib.register("fb_count_valid", [vp, i64, i32, vp, vp])
_lib.register("fb_cross_entropy", [vp, vp, vp, vp, vp, f32, i64, i32, i64, i32, i32, vp])
_lib.register("fb_cross_entropy_opt", [vp, vp, vp, vp, vp, f32, i64, i32, i64, i32, i32, f32, f32, f32, f32, vp])
_lib.register("fb_mean_loss", [vp, i64, vp, vp, i32, vp])


class CEOptions:
    """The loss options of the reference's fused cross-entropy (fla/modules/fused_cross_entropy.py:374-400): the loss is
    taken on ``z = softcap * tanh(logit_scale * x / softcap)`` (no soft-capping: ``z = logit_scale * x``) as
    ``lse(z) - smoothing * mean(z) - (1 - smoothing) * z_target + lse_square_scale * lse(z)**2``."""

    __slots__ = ("label_smoothing", "logit_scale", "lse_square_scale", "logit_softcapping")

    def __init__(self, label_smoothing: float = 0.0, logit_scale: float = 1.0, lse_square_scale: float = 0.0,
                 logit_softcapping: Optional[float] = None) -> None:
        self.label_smoothing, self.logit_scale = float(label_smoothing), float(logit_scale)
        self.lse_square_scale = float(lse_square_scale)
        self.logit_softcapping = float(logit_softcapping) if logit_softcapping else 0.0

    def args(self):
        return (self.label_smoothing, self.logit_scale, self.lse_square_scale, self.logit_softcapping)

    @property
    def plain(self) -> bool:
        return self.args() == (0.0, 1.0, 0.0, 0.0)


_PLAIN = CEOptions()


def cross_entropy_reference(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                            opt: CEOptions = _PLAIN) -> torch.Tensor:
    """The same loss written out with torch ops in fp32 (the oracle of the kernel tests, and the CPU path)."""
    z = logits.float() * opt.logit_scale
    if opt.logit_softcapping > 0:
        z = opt.logit_softcapping * torch.tanh(z / opt.logit_softcapping)
    lse = torch.logsumexp(z, -1)
    valid = labels != ignore_index
    tgt = z.gather(-1, labels.clamp_min(0).unsqueeze(-1)).squeeze(-1)
    rows = lse - opt.label_smoothing * z.mean(-1) - (1.0 - opt.label_smoothing) * tgt + opt.lse_square_scale * lse * lse
    rows = torch.where(valid, rows, torch.zeros_like(rows))
    return rows.sum() / valid.sum().clamp_min(1)


def _kernel_ok(x: torch.Tensor) -> bool:
    return _lib.available() and x.is_cuda and x.dtype == torch.bfloat16


class _FLCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, labels, ignore_index, chunk, grad_scale, opt=_PLAIN):
        L = _lib.lib()
        T, D = x.shape
        V = weight.shape[0]
        dev = x.device
        stream = _lib.stream_ptr()
        labels = labels.contiguous()
        n_valid = torch.empty(1, dtype=torch.int32, device=dev)
        _lib.check(L.fb_count_valid(labels.data_ptr(), T, ignore_index, n_valid.data_ptr(), stream), "fb_count_valid")
        loss_rows = torch.empty(T, dtype=torch.float32, device=dev)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        need_grad = x.requires_grad or weight.requires_grad
        dx = torch.empty_like(x) if need_grad else None
        mg = getattr(weight, "main_grad", None)
        dw = None
        if need_grad and mg is None:
            dw = torch.zeros(V, D, dtype=torch.float32, device=dev)
        wgrad_out = mg if mg is not None else dw
        C = min(chunk, T)
        logits = torch.empty(C, V, dtype=torch.bfloat16, device=dev)
        launches = 2
        for a in range(0, T, C):
            b = min(T, a + C)
            n = b - a
            lg = logits[:n]
            gemm_nt(x[a:b], weight.detach(), out=lg)
            rc = L.fb_cross_entropy_opt(lg.data_ptr(), labels[a:b].data_ptr(), loss_rows[a:b].data_ptr(), 0,
                                        n_valid.data_ptr(), float(grad_scale), n, V, lg.stride(0), ignore_index,
                                        1 if need_grad else 0, *opt.args(), stream)
            _lib.check(rc, "fb_cross_entropy")
            launches += 1
            if need_grad:
                gemm_nn(lg, weight.detach(), out=dx[a:b])
                gemm_tn(lg, x[a:b], out=wgrad_out, accumulate=True)
        _lib.check(L.fb_mean_loss(loss_rows.data_ptr(), T, n_valid.data_ptr(), loss.data_ptr(), 0, stream), "fb_mean_loss")
        _lib.count_launch(launches)
        ctx.save_for_backward(dx, dw)
        ctx.grad_scale = grad_scale
        ctx.has_main_grad = mg is not None
        return loss[0]

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        # Gradients were formed in the forward with d(loss) = grad_scale.  With a main_grad weight the incoming
        # dloss must be 1 (the trainer passes its 1/accumulation factor as grad_scale instead).
        gx = dx * dloss.to(dx.dtype) if dx is not None else None
        gw = None
        if dw is not None:
            gw = (dw * dloss).to(torch.bfloat16)
        return gx, gw, None, None, None, None, None


def fused_linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                               chunk: int = 8192, grad_scale: float = 1.0, label_smoothing: float = 0.0,
                               logit_scale: float = 1.0, lse_square_scale: float = 0.0,
                               logit_softcapping: Optional[float] = None) -> torch.Tensor:
    """Mean cross-entropy of ``x @ weight.T`` against ``labels`` over non-ignored positions (fp32 scalar); the keyword
    options are those of ``CEOptions``."""
    x2 = x.reshape(-1, x.shape[-1])
    lab = labels.reshape(-1)
    opt = CEOptions(label_smoothing, logit_scale, lse_square_scale, logit_softcapping)
    if _kernel_ok(x2) and weight.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0:
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        return _FLCEFn.apply(x2, weight, lab, ignore_index, chunk, grad_scale, opt)
    logits = F.linear(x2, weight).float()
    loss = F.cross_entropy(logits, lab, ignore_index=ignore_index) if opt.plain else \
        cross_entropy_reference(logits, lab, ignore_index, opt)
    if grad_scale != 1.0:
        # same value, gradient scaled by grad_scale (matches the kernel path's contract)
        loss = loss.detach() + (loss - loss.detach()) * grad_scale
    return loss


class _CEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, opt=_PLAIN):
        L = _lib.lib()
        T, V = logits.shape
        dev = logits.device
        stream = _lib.stream_ptr()
        labels = labels.contiguous()
        n_valid = torch.empty(1, dtype=torch.int32, device=dev)
        _lib.check(L.fb_count_valid(labels.data_ptr(), T, ignore_index, n_valid.data_ptr(), stream), "fb_count_valid")
        loss_rows = torch.empty(T, dtype=torch.float32, device=dev)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        # in-place backward: the logits buffer becomes the gradient (inplace_backward=True in the reference)
        rc = L.fb_cross_entropy_opt(logits.data_ptr(), labels.data_ptr(), loss_rows.data_ptr(), 0, n_valid.data_ptr(), 1.0,
                                    T, V, logits.stride(0), ignore_index, 1 if logits.requires_grad else 0, *opt.args(),
                                    stream)
        _lib.check(rc, "fb_cross_entropy")
        _lib.check(L.fb_mean_loss(loss_rows.data_ptr(), T, n_valid.data_ptr(), loss.data_ptr(), 0, stream), "fb_mean_loss")
        _lib.count_launch(3)
        ctx.save_for_backward(logits)
        return loss[0]

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return g * dloss.to(g.dtype), None, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, label_smoothing: float = 0.0,
                  logit_scale: float = 1.0, lse_square_scale: float = 0.0,
                  logit_softcapping: Optional[float] = None) -> torch.Tensor:
    """Row-wise cross-entropy with in-place gradient on the GPU; keyword options as in ``CEOptions``."""
    lg = logits.reshape(-1, logits.shape[-1])
    lab = labels.reshape(-1)
    opt = CEOptions(label_smoothing, logit_scale, lse_square_scale, logit_softcapping)
    if _kernel_ok(lg) and lg.is_contiguous() and lg.shape[-1] % 8 == 0:
        return _CEFn.apply(lg, lab, ignore_index, opt)
    if opt.plain:
        return F.cross_entropy(lg.float(), lab, ignore_index=ignore_index)
    return cross_entropy_reference(lg, lab, ignore_index, opt)
