"""ctypes wrappers of the CUDA-core helper kernels of the chunk algorithms (``csrc/chunk.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import _lib

_lib.register("fb_tri_inverse", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p])
_lib.register("fb_state_step", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])


def tri_inverse(A: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``(I + A)^-1`` for strictly lower-triangular fp32 ``A [..., 64, 64]``."""
    assert A.shape[-1] == 64 and A.shape[-2] == 64 and A.dtype == torch.float32
    A = A.contiguous()
    out = torch.empty(A.shape, dtype=out_dtype, device=A.device)
    n = A.numel() // 4096
    o16, o32 = (out.data_ptr(), 0) if out_dtype == torch.bfloat16 else (0, out.data_ptr())
    _lib.check(_lib.lib().fb_tri_inverse(A.data_ptr(), o16, o32, n, _lib.stream_ptr()), "fb_tri_inverse")
    _lib.count_launch()
    return out


def state_step(idx: torch.Tensor, alpha: torch.Tensor, X: torch.Tensor, X16: torch.Tensor, reverse: bool) -> None:
    """One chunk position of ``X[c+1] = alpha_c X[c] + X[c+1]`` (or its reverse) for the chunks in ``idx``."""
    _, H, rows, cols = X.shape
    per_row = 1 if alpha.dim() == 3 else 0
    rc = _lib.lib().fb_state_step(idx.data_ptr(), idx.numel(), alpha.data_ptr(), per_row, X.data_ptr(), X16.data_ptr(), H,
                                  rows, cols, int(reverse), _lib.stream_ptr())
    _lib.check(rc, "fb_state_step")
    _lib.count_launch()


_lib.register("fb_gla_diag_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
_lib.register("fb_gla_diag_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_float, c_void_p])


def gla_diag_fwd(q: torch.Tensor, k: torch.Tensor, b: torch.Tensor, scale: float, A: torch.Tensor) -> None:
    """Writes the four diagonal 16 x 16 sub-blocks of ``A [NC, H, 64, 64]`` (fp32); q, k ``[NC, 64, H, dk]`` bf16,
    b ``[NC, 64, H, dk]`` fp32, all contiguous."""
    NC, _, H, dk = q.shape
    rc = _lib.lib().fb_gla_diag_fwd(q.data_ptr(), k.data_ptr(), b.data_ptr(), A.data_ptr(), NC, H, dk, float(scale),
                                    _lib.stream_ptr())
    _lib.check(rc, "fb_gla_diag_fwd")
    _lib.count_launch()


def gla_diag_bwd(q, k, b, dA, dq, dk_, db, scale: float) -> None:
    """Adds the diagonal sub-blocks' gradient contributions into fp32 ``dq, dk, db [NC, 64, H, dk]``."""
    NC, _, H, dk = q.shape
    rc = _lib.lib().fb_gla_diag_bwd(q.data_ptr(), k.data_ptr(), b.data_ptr(), dA.data_ptr(), dq.data_ptr(), dk_.data_ptr(),
                                    db.data_ptr(), NC, H, dk, float(scale), _lib.stream_ptr())
    _lib.check(rc, "fb_gla_diag_bwd")
    _lib.count_launch()


_lib.register("fb_l2norm_fwd", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_void_p])
_lib.register("fb_l2norm_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p])


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        xc = x.contiguous()
        D = xc.shape[-1]
        rows = xc.numel() // D
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().fb_l2norm_fwd(xc.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, D, float(eps),
                                            _lib.stream_ptr()), "fb_l2norm_fwd")
        _lib.count_launch()
        ctx.save_for_backward(xc, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        D = xc.shape[-1]
        dx = torch.empty_like(xc)
        _lib.check(_lib.lib().fb_l2norm_bwd(xc.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dx.data_ptr(), xc.numel() // D, D,
                                            _lib.stream_ptr()), "fb_l2norm_bwd")
        _lib.count_launch()
        return dx, None


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(sum(x^2, -1) + eps)`` for bf16 ``x [..., D]``, D <= 1024 (fla/modules/l2norm.py)."""
    return _L2Norm.apply(x, eps)


_lib.register("fb_pair_dot", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])


def pair_dot(x: torch.Tensor, y: torch.Tensor, per_row: bool) -> torch.Tensor:
    """fp32 ``sum(x * y)`` over the last two dims (``per_row``: the last dim) of bf16 ``[..., R, C]`` tensors."""
    x, y = x.contiguous(), y.contiguous()
    R, C = x.shape[-2:]
    B = x.numel() // (R * C)
    out = torch.empty(*x.shape[:-2], *([R] if per_row else []), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().fb_pair_dot(x.data_ptr(), y.data_ptr(), out.data_ptr(), B, R, C, int(per_row), _lib.stream_ptr()),
               "fb_pair_dot")
    _lib.count_launch()
    return out


_lib.register("fb_state_scan", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_void_p])


def state_scan(first: torch.Tensor, last: torch.Tensor, alpha: torch.Tensor, X: torch.Tensor, X16: torch.Tensor,
               reverse: bool) -> None:
    """The whole recurrence ``X[c+1] = alpha_c X[c] + X[c+1]`` (or its reverse) of every document in one launch;
    ``first`` / ``last`` are the int64 chunk ranges of the documents."""
    _, H, rows, cols = X.shape
    per_row = 1 if alpha.dim() == 3 else 0
    rc = _lib.lib().fb_state_scan(first.data_ptr(), last.data_ptr(), first.numel(), alpha.data_ptr(), per_row, X.data_ptr(),
                                  X16.data_ptr(), H, rows, cols, int(reverse), _lib.stream_ptr())
    _lib.check(rc, "fb_state_scan")
    _lib.count_launch()


_lib.register("fb_gla_prep_fwd", [c_void_p] * 9 + [c_int, c_int, c_int, c_float, c_void_p])
_lib.register("fb_gla_prep_bwd", [c_void_p] * 12 + [c_int, c_int, c_int, c_float, c_void_p])


class GlaPrep(torch.autograd.Function):
    """One pass over a chunk's q, k, g producing the cumulative decay and every scaled operand of the GLA chunk
    algorithm (see ``csrc/chunk.cu: gla_prep_fwd_kernel``).  q, k ``[NC, 64, H, dk]`` bf16, g ``[NC, 64, H, dk]`` fp32.
    Returns ``(b, khat, qbar, qt, k3, alpha)``."""

    @staticmethod
    def forward(ctx, qp, kp, gp, scale):
        qp, kp, gp = qp.contiguous(), kp.contiguous(), gp.contiguous()
        NC, C, H, dk = qp.shape
        assert C == 64 and qp.dtype == torch.bfloat16 and gp.dtype == torch.float32
        dev = qp.device
        b = torch.empty_like(gp)
        khat, qbar, qt = torch.empty_like(kp), torch.empty_like(qp), torch.empty_like(qp)
        k3 = torch.empty(NC, 3, 48, H, dk, dtype=torch.bfloat16, device=dev)
        alpha = torch.empty(NC, H, dk, dtype=torch.float32, device=dev)
        rc = _lib.lib().fb_gla_prep_fwd(qp.data_ptr(), kp.data_ptr(), gp.data_ptr(), b.data_ptr(), khat.data_ptr(),
                                        qbar.data_ptr(), qt.data_ptr(), k3.data_ptr(), alpha.data_ptr(), NC, H, dk,
                                        float(scale), _lib.stream_ptr())
        _lib.check(rc, "fb_gla_prep_fwd")
        _lib.count_launch()
        ctx.save_for_backward(qp, kp, b)
        ctx.scale = scale
        return b, khat, qbar, qt, k3, alpha

    @staticmethod
    def backward(ctx, db, dkhat, dqbar, dqt, dk3, dalpha):
        qp, kp, b = ctx.saved_tensors
        NC, C, H, dk = qp.shape

        def c16(t):
            return None if t is None else t.to(torch.bfloat16).contiguous()

        def c32(t):
            return None if t is None else t.float().contiguous()
        dkhat, dqbar, dqt, dk3 = c16(dkhat), c16(dqbar), c16(dqt), c16(dk3)
        db, dalpha = c32(db), c32(dalpha)
        dq, dk_ = torch.empty_like(qp), torch.empty_like(kp)
        dg = torch.empty_like(b)
        rc = _lib.lib().fb_gla_prep_bwd(qp.data_ptr(), kp.data_ptr(), b.data_ptr(), _lib.ptr(dkhat), _lib.ptr(dqbar),
                                        _lib.ptr(dqt), _lib.ptr(dk3), _lib.ptr(dalpha), _lib.ptr(db), dq.data_ptr(),
                                        dk_.data_ptr(), dg.data_ptr(), NC, H, dk, float(ctx.scale), _lib.stream_ptr())
        _lib.check(rc, "fb_gla_prep_bwd")
        _lib.count_launch()
        return dq, dk_, dg, None


_lib.register("fb_scalar_prep_fwd", [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_float, c_void_p])
_lib.register("fb_scalar_prep_bwd", [c_void_p] * 10 + [c_int, c_int, c_int, c_int, c_float, c_void_p])


def scalar_prep_supported(C: int, dk: int) -> bool:
    n = dk // 8
    return C in (64, 128) and dk % 8 == 0 and n > 0 and (n & (n - 1)) == 0


class ScalarPrep(torch.autograd.Function):
    """Cumulative decay and the two token-sized scalings of the scalar-gated chunk algorithms in one kernel:
    ``b = cumsum(g)``, ``khat = k e^{b_last - b}``, ``qbar = scale q e^{b}``, ``alpha = e^{b_last}``.
    q, k ``[NC, C, H, dk]`` bf16, g ``[NC, C, H]`` fp32 or None.  Returns ``(b, khat, qbar, alpha)``."""

    @staticmethod
    def forward(ctx, qp, kp, gp, scale):
        qp, kp = qp.contiguous(), kp.contiguous()
        NC, C, H, dk = qp.shape
        dev = qp.device
        if gp is not None:
            gp = gp.float().contiguous()
        b = torch.empty(NC, C, H, dtype=torch.float32, device=dev)
        khat, qbar = torch.empty_like(kp), torch.empty_like(qp)
        alpha = torch.empty(NC, H, dtype=torch.float32, device=dev)
        rc = _lib.lib().fb_scalar_prep_fwd(qp.data_ptr(), kp.data_ptr(), _lib.ptr(gp), b.data_ptr(), khat.data_ptr(),
                                           qbar.data_ptr(), alpha.data_ptr(), NC, C, H, dk, float(scale), _lib.stream_ptr())
        _lib.check(rc, "fb_scalar_prep_fwd")
        _lib.count_launch()
        ctx.save_for_backward(qp, kp, b)
        ctx.scale = scale
        ctx.has_g = gp is not None
        return b, khat, qbar, alpha

    @staticmethod
    def backward(ctx, db, dkhat, dqbar, dalpha):
        qp, kp, b = ctx.saved_tensors
        NC, C, H, dk = qp.shape
        dkhat = None if dkhat is None else dkhat.to(torch.bfloat16).contiguous()
        dqbar = None if dqbar is None else dqbar.to(torch.bfloat16).contiguous()
        db = None if db is None else db.float().contiguous()
        dalpha = None if dalpha is None else dalpha.float().contiguous()
        dq, dk_ = torch.empty_like(qp), torch.empty_like(kp)
        dg = torch.empty_like(b)
        rc = _lib.lib().fb_scalar_prep_bwd(qp.data_ptr(), kp.data_ptr(), b.data_ptr(), _lib.ptr(dkhat), _lib.ptr(dqbar),
                                           _lib.ptr(dalpha), _lib.ptr(db), dq.data_ptr(), dk_.data_ptr(), dg.data_ptr(), NC,
                                           C, H, dk, float(ctx.scale), _lib.stream_ptr())
        _lib.check(rc, "fb_scalar_prep_bwd")
        _lib.count_launch()
        return dq, dk_, (dg if ctx.has_g else None), None


_lib.register("fb_sscan_fwd", [c_void_p] * 8 + [c_int] + [c_void_p] * 4 + [c_int, c_int, c_int, c_void_p])
_lib.register("fb_sscan_bwd", [c_void_p] * 9 + [c_int] + [c_void_p] * 10 + [c_int, c_int, c_int, c_void_p])
_lib.register("fb_sscan_channel_blocks", [c_int])


class SelectiveScan(torch.autograd.Function):
    """Mamba-1 selective scan on the chunk-parallel kernels of ``csrc/sscan.cu``.  Inputs in the 64-token chunk layout:
    u ``[NC, 64, Di]`` bf16, delta ``[NC, 64, Di]`` fp32, A ``[Di, 16]`` fp32, B, C ``[NC, 64, 16]`` fp32, D ``[Di]`` fp32;
    ``first`` / ``last``: int64 chunk range of every document.  Returns y ``[NC, 64, Di]`` bf16."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, first, last):
        u, delta, A, B, C, D = (t.contiguous() for t in (u, delta, A, B, C, D))
        NC, L, Di = u.shape
        N = A.shape[1]
        assert L == 64 and N == 16 and u.dtype == torch.bfloat16
        dev = u.device
        hloc = torch.empty(NC, Di, N, dtype=torch.float32, device=dev)
        P, hin = torch.empty_like(hloc), torch.empty_like(hloc)
        y = torch.empty_like(u)
        rc = _lib.lib().fb_sscan_fwd(u.data_ptr(), delta.data_ptr(), A.data_ptr(), B.data_ptr(), C.data_ptr(), D.data_ptr(),
                                     first.data_ptr(), last.data_ptr(), first.numel(), hloc.data_ptr(), P.data_ptr(),
                                     hin.data_ptr(), y.data_ptr(), NC, Di, N, _lib.stream_ptr())
        _lib.check(rc, "fb_sscan_fwd")
        _lib.count_launch(3)
        ctx.save_for_backward(u, delta, A, B, C, D, first, last, P, hin)
        return y

    @staticmethod
    def backward(ctx, dy):
        u, delta, A, B, C, D, first, last, P, hin = ctx.saved_tensors
        NC, L, Di = u.shape
        N = A.shape[1]
        dev = u.device
        dy = dy.to(torch.bfloat16).contiguous()
        gloc, gout = torch.empty_like(P), torch.empty_like(P)
        du = torch.empty(NC, L, Di, dtype=torch.float32, device=dev)
        ddl = torch.empty_like(du)
        nblk = int(_lib.lib().fb_sscan_channel_blocks(Di))
        dA = torch.empty(NC, Di, N, dtype=torch.float32, device=dev)      # per-chunk partials, summed below
        dB = torch.empty(nblk, NC, L, N, dtype=torch.float32, device=dev)  # per-channel-block partials
        dC = torch.empty_like(dB)
        dD = torch.empty(NC, Di, dtype=torch.float32, device=dev)
        rc = _lib.lib().fb_sscan_bwd(u.data_ptr(), delta.data_ptr(), A.data_ptr(), B.data_ptr(), C.data_ptr(), D.data_ptr(),
                                     dy.data_ptr(), first.data_ptr(), last.data_ptr(), first.numel(), P.data_ptr(),
                                     hin.data_ptr(), gloc.data_ptr(), gout.data_ptr(), du.data_ptr(), ddl.data_ptr(),
                                     dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), dD.data_ptr(), NC, Di, N, _lib.stream_ptr())
        _lib.check(rc, "fb_sscan_bwd")
        _lib.count_launch(3)
        return du.to(u.dtype), ddl, dA.sum(0), dB.sum(0), dC.sum(0), dD.sum(0), None, None


_lib.register("fb_vdecay_diag_fwd", [c_void_p] * 4 + [c_int, c_int, c_int, c_void_p])
_lib.register("fb_vdecay_diag_bwd", [c_void_p] * 7 + [c_int, c_int, c_int, c_void_p])


class VdecayDiag(torch.autograd.Function):
    """Diagonal 16 x 16 sub-blocks of the value-decayed intra-chunk product (``csrc/chunk.cu: vdecay_diag_*``):
    P ``[NC, H, 64, 64]`` fp32, v ``[NC, 64, H, M]`` bf16, b ``[NC, 64, H, M]`` fp32 -> ``[NC, 64, H, M]`` fp32."""

    @staticmethod
    def forward(ctx, P, v, b):
        P, v, b = P.float().contiguous(), v.contiguous(), b.contiguous()
        NC, C, H, M = v.shape
        assert C == 64 and v.dtype == torch.bfloat16
        o = torch.empty(NC, C, H, M, dtype=torch.float32, device=v.device)
        _lib.check(_lib.lib().fb_vdecay_diag_fwd(P.data_ptr(), v.data_ptr(), b.data_ptr(), o.data_ptr(), NC, H, M,
                                                 _lib.stream_ptr()), "fb_vdecay_diag_fwd")
        _lib.count_launch()
        ctx.save_for_backward(P, v, b)
        return o

    @staticmethod
    def backward(ctx, do):
        P, v, b = ctx.saved_tensors
        NC, C, H, M = v.shape
        do = do.float().contiguous()
        dP = torch.zeros_like(P)
        dv = torch.empty(NC, C, H, M, dtype=torch.float32, device=v.device)
        db = torch.empty_like(dv)
        _lib.check(_lib.lib().fb_vdecay_diag_bwd(P.data_ptr(), v.data_ptr(), b.data_ptr(), do.data_ptr(), dP.data_ptr(),
                                                 dv.data_ptr(), db.data_ptr(), NC, H, M, _lib.stream_ptr()), "fb_vdecay_diag_bwd")
        _lib.count_launch()
        return dP, dv.to(v.dtype), db


_lib.register("fb_scores_bwd_prep", [c_void_p] * 5 + [c_longlong] * 3 + [c_int] * 4 + [c_void_p, c_void_p, c_void_p])


def scores_bwd_prep(dc: torch.Tensor, out: torch.Tensor, d: torch.Tensor, mask_mode: int):
    """For score blocks ``out = alpha (a b^T) exp(d_i - d_j)`` (masked): returns the bf16 GEMM operand
    ``dc * keep * exp(d_i - d_j)`` and the fp32 gradient of ``d``.  dc, out ``[NC, H, C, C]`` (fp32 or bf16),
    d ``[NC, H, C]`` fp32 with any strides."""
    NC, H, C, _ = out.shape
    dc, out = dc.contiguous(), out.contiguous()
    g = torch.empty(NC, H, C, C, dtype=torch.bfloat16, device=out.device)
    dd = torch.empty(NC, H, C, dtype=torch.float32, device=out.device)
    dc32, dc16 = (dc.data_ptr(), 0) if dc.dtype == torch.float32 else (0, dc.to(torch.bfloat16).data_ptr())
    c32, c16 = (out.data_ptr(), 0) if out.dtype == torch.float32 else (0, out.data_ptr())
    if dc.dtype not in (torch.float32, torch.bfloat16):
        dc = dc.float()
        dc32, dc16 = dc.data_ptr(), 0
    dh, dl, dr = d.stride()
    rc = _lib.lib().fb_scores_bwd_prep(dc32, dc16, c32, c16, d.data_ptr(), dh, dl, dr, NC, H, C, int(mask_mode), g.data_ptr(),
                                       dd.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "fb_scores_bwd_prep")
    _lib.count_launch()
    return g, dd
