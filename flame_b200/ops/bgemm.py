"""Batched bf16 GEMM over (chunk, head) batches on the tcgen05 kernel of ``csrc/bgemm.cu``.

Every operand is a 4-D view ``[hi, lo, rows, inner]`` (inner stride 1, any other strides), which is what a
``permute`` of the chunk layout ``[chunks, 64, heads, d]`` gives, so no operand is ever copied or transposed:

* ``mn=False``: rows are the operand's M (or N) dimension and inner is K;
* ``mn=True``:  rows are K and inner is the M (or N) dimension.

``bgemm`` computes ``C[b] = alpha * A[b] @ B[b]^T`` with the epilogue options the chunk algorithms need (causal
masks, the decay factor ``exp(d[row] - d[col])``, the state step ``C = acc + gamma * Cin (+ C)`` and a bf16
mirror).  ``bmm`` is the differentiable plain product built on it.  Without CUDA the same functions run on
``torch.matmul`` so that the chunk algorithms are testable on CPU.

Stands in for the ``tl.dot`` bodies of the reference's chunk kernels (fla/ops/common/chunk_h.py,
fla/ops/common/chunk_o.py, fla/ops/gated_delta_rule/wy_fast.py).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib


class _Operand(ctypes.Structure):
    _fields_ = [("ptr", c_void_p), ("ld", c_longlong), ("stride_lo", c_longlong), ("stride_hi", c_longlong),
                ("n_lo", c_int), ("n_hi", c_int), ("mn", c_int), ("lo_div", c_int), ("hi_offset", c_int),
                ("hi_index", c_void_p)]


class _Epilogue(ctypes.Structure):
    _fields_ = [("C", c_void_p), ("ldc", c_longlong), ("stride_lo", c_longlong), ("stride_hi", c_longlong),
                ("c_lo_div", c_int), ("c_hi_offset", c_int), ("c_hi_index", c_void_p),
                ("Cin", c_void_p), ("cin_hi_offset", c_int), ("cin_hi_index", c_void_p), ("gamma", c_void_p),
                ("C16", c_void_p), ("c16_hi_offset", c_int), ("c16_hi_index", c_void_p),
                ("add16", c_void_p), ("add16_hi_offset", c_int), ("add16_hi_index", c_void_p),
                ("ld16", c_longlong), ("stride_lo16", c_longlong), ("stride_hi16", c_longlong),
                ("decay", c_void_p), ("d_hi", c_longlong), ("d_lo", c_longlong), ("d_r", c_longlong),
                ("alpha", c_float), ("out_mode", c_int), ("mask_mode", c_int)]


_lib.register("fb_bgemm_bf16", [POINTER(_Operand), POINTER(_Operand), POINTER(_Epilogue), c_int, c_int, c_int, c_int,
                                c_int, c_void_p])

MASK_NONE, MASK_TRIL, MASK_STRICT = 0, 1, 2


def _use_kernel(*ts: torch.Tensor) -> bool:
    return _lib.available() and all(t.is_cuda for t in ts)


def _inner_contig(t: torch.Tensor) -> torch.Tensor:
    """Kernel operands need inner stride 1, 16-byte aligned rows/batches and no broadcast (stride 0) batch dims."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 and s > 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _operand(t: torch.Tensor, mn: bool, lo_div: int, index: Optional[torch.Tensor], offset: int) -> _Operand:
    return _Operand(t.data_ptr(), t.stride(2), t.stride(1), t.stride(0), t.shape[1], t.shape[0], int(mn), lo_div, offset,
                    _lib.ptr(index))


def _mkn(a, b, a_mn, b_mn):
    M, K = (a.shape[3], a.shape[2]) if a_mn else (a.shape[2], a.shape[3])
    N, Kb = (b.shape[3], b.shape[2]) if b_mn else (b.shape[2], b.shape[3])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    return M, N, K


def _mask(M, N, mode, device):
    r = torch.arange(M, device=device)[:, None]
    c = torch.arange(N, device=device)[None, :]
    return (c <= r) if mode == MASK_TRIL else (c < r)


def bgemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
          out_dtype: Optional[torch.dtype] = None, alpha: float = 1.0, mask: int = MASK_NONE,
          decay: Optional[torch.Tensor] = None, accumulate: bool = False, cin: Optional[torch.Tensor] = None,
          gamma: Optional[torch.Tensor] = None, out16: Optional[torch.Tensor] = None,
          a_index: Optional[torch.Tensor] = None, b_index: Optional[torch.Tensor] = None,
          c_index: Optional[torch.Tensor] = None, cin_index: Optional[torch.Tensor] = None, c_offset: int = 0,
          cin_offset: int = 0, a_offset: int = 0, b_offset: int = 0, n_hi: Optional[int] = None,
          n_lo: Optional[int] = None, out16_index: Optional[torch.Tensor] = None, out16_offset: int = 0,
          add16: Optional[torch.Tensor] = None, add16_index: Optional[torch.Tensor] = None,
          add16_offset: int = 0) -> torch.Tensor:
    """``out[hi, lo] = alpha * a[hi, lo] @ b[hi, lo]^T`` (no autograd).

    ``a``/``b``: ``[hi, lo, rows, inner]`` bf16 views.  ``n_lo`` defaults to the larger head count; an operand with
    fewer heads is shared by ``n_lo / heads`` consecutive batches.  ``*_index`` (int32 ``[n_hi]``) select the hi
    coordinate per batch; ``c_offset`` / ``cin_offset`` are added to the output / addend hi coordinate.
    ``decay``: fp32 ``[hi, lo, M]`` (any strides): values are multiplied by ``exp(d[row] - d[col])`` where kept.
    ``cin`` (fp32, layout of ``out``; may be ``out`` itself for an in-place state) is added scaled by
    ``gamma[hi(a), lo]``; ``add16`` (bf16) is added; ``out16`` receives a bf16 copy.  ``out16`` and ``add16`` are
    ``[*, lo, M, N]`` tensors with hi coordinates of their own (index / offset; default: the batch number).
    """
    M, N, K = _mkn(a, b, a_mn, b_mn)
    n_lo = n_lo or max(a.shape[1], b.shape[1])
    if n_hi is None:
        n_hi = len(a_index) if a_index is not None else (len(b_index) if b_index is not None else min(a.shape[0], b.shape[0]))
    if out is None:
        assert c_index is None and c_offset == 0
        out = torch.empty(n_hi, n_lo, M, N, dtype=out_dtype or a.dtype, device=a.device)
    assert out.shape[2:] == (M, N) and out.stride(-1) == 1, (out.shape, out.stride())
    if accumulate or cin is not None or out16 is not None:
        assert out.dtype == torch.float32
    if n_hi == 0:
        return out
    if _use_kernel(a, b):
        a = _inner_contig(a)
        b = _inner_contig(b)
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        ea = _operand(a, a_mn, n_lo // a.shape[1], a_index, a_offset)
        eb = _operand(b, b_mn, n_lo // b.shape[1], b_index, b_offset)
        if cin is not None:
            assert cin.dtype == torch.float32 and cin.stride() == out.stride()
        side = out16 if out16 is not None else add16
        ld16 = slo16 = shi16 = 0
        if side is not None:
            assert side.dtype == torch.bfloat16 and side.stride(-1) == 1
            shi16, slo16, ld16 = side.stride()[:3]
            if out16 is not None and add16 is not None:
                assert add16.dtype == torch.bfloat16 and add16.stride()[1:] == out16.stride()[1:]
                assert add16.stride(0) == out16.stride(0)
        if gamma is not None:
            assert gamma.dtype == torch.float32 and gamma.is_contiguous() and gamma.shape[-1] == n_lo
        d_hi = d_lo = d_r = 0
        if decay is not None:
            assert decay.dtype == torch.float32 and decay.shape[-1] == M == N
            d_hi, d_lo, d_r = decay.stride()
        mode = 0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
        ep = _Epilogue(out.data_ptr(), out.stride(2), out.stride(1), out.stride(0), n_lo // out.shape[1], c_offset,
                       _lib.ptr(c_index), _lib.ptr(cin), cin_offset, _lib.ptr(cin_index), _lib.ptr(gamma),
                       _lib.ptr(out16), out16_offset, _lib.ptr(out16_index), _lib.ptr(add16), add16_offset,
                       _lib.ptr(add16_index), ld16, slo16, shi16,
                       _lib.ptr(decay), d_hi, d_lo, d_r, float(alpha), mode, int(mask))
        rc = _lib.lib().fb_bgemm_bf16(ctypes.byref(ea), ctypes.byref(eb), ctypes.byref(ep), n_hi, n_lo, M, N, K,
                                      _lib.stream_ptr())
        _lib.check(rc, "fb_bgemm_bf16")
        _lib.count_launch()
        return out
    # ---- reference path
    dev = a.device

    def pick(t, index, div, off):
        t = t[off:off + n_hi] if index is None else t[index.long() + off]
        return t.repeat_interleave(div, dim=1) if div > 1 else t

    af = pick(a, a_index, n_lo // a.shape[1], a_offset).float()
    bf = pick(b, b_index, n_lo // b.shape[1], b_offset).float()
    af = af.transpose(-1, -2) if a_mn else af
    bf = bf if b_mn else bf.transpose(-1, -2)
    r = torch.matmul(af, bf) * alpha
    if decay is not None:
        d = decay[:n_hi].float()
        r = r * (d[..., :, None] - d[..., None, :]).clamp_max(0.0 if mask else 80.0).exp()
    if mask:
        r = r.masked_fill(~_mask(M, N, mask, dev), 0.0)
    hi_c = (torch.arange(n_hi, device=dev) if c_index is None else c_index.long()) + c_offset
    if accumulate:
        r = r + out[hi_c].float()
    if cin is not None:
        hi_in = (torch.arange(n_hi, device=dev) if cin_index is None else cin_index.long()) + cin_offset
        g = 1.0
        if gamma is not None:
            hi_a = torch.arange(n_hi, device=dev) if a_index is None else a_index.long()
            g = gamma[hi_a][..., None, None]
        r = r + g * cin[hi_in]
    if add16 is not None:
        hi_add = (torch.arange(n_hi, device=dev) if add16_index is None else add16_index.long()) + add16_offset
        r = r + add16[hi_add].float()
    out[hi_c] = r.to(out.dtype)
    if out16 is not None:
        hi_16 = (torch.arange(n_hi, device=dev) if out16_index is None else out16_index.long()) + out16_offset
        out16[hi_16] = r.to(out16.dtype)
    return out


def _empty_like_layout(t: torch.Tensor, dtype=None) -> torch.Tensor:
    """An uninitialised tensor with the shape and (dense) stride order of ``t``."""
    if t.is_contiguous() or t.stride(-1) != 1:
        return torch.empty(t.shape, dtype=dtype or t.dtype, device=t.device)
    order = sorted(range(t.dim()), key=lambda i: (t.stride(i), -i), reverse=True)
    shape = [t.shape[i] for i in order]
    base = torch.empty(shape, dtype=dtype or t.dtype, device=t.device)
    inv = [order.index(i) for i in range(t.dim())]
    return base.permute(inv)


class _BMM(torch.autograd.Function):
    """Differentiable ``alpha * A @ B^T (+ addend)`` over 4-D operands; gradients come back in the operands' own layouts."""

    @staticmethod
    def forward(ctx, a, b, a_mn, b_mn, alpha, token_major, out_dtype, addend=None):
        M, N, K = _mkn(a, b, a_mn, b_mn)
        n_lo = max(a.shape[1], b.shape[1])
        n_hi = a.shape[0]
        out_dtype = out_dtype or a.dtype
        if token_major:
            out = torch.empty(n_hi, M, n_lo, N, dtype=out_dtype, device=a.device).permute(0, 2, 1, 3)
        else:
            out = torch.empty(n_hi, n_lo, M, N, dtype=out_dtype, device=a.device)
        if addend is not None and _use_kernel(a, b) and out.dtype == torch.bfloat16 and addend.dtype == torch.bfloat16 \
                and addend.stride() == out.stride():
            bgemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, alpha=alpha, add16=addend)
        else:
            bgemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, alpha=alpha)
            if addend is not None:
                out += addend
        ctx.save_for_backward(a, b)
        ctx.cfg = (a_mn, b_mn, alpha)
        ctx.has_addend = addend is not None
        return out

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        a_mn, b_mn, alpha = ctx.cfg
        dc = dc if dc.dtype == a.dtype else dc.to(a.dtype)
        n_lo = dc.shape[1]
        da = db = None
        if ctx.needs_input_grad[0]:
            ga = _empty_like_layout(a) if a.shape[1] == n_lo else None
            if ga is None:  # shared (grouped) heads: reduce over the group afterwards
                full = torch.empty(a.shape[0], n_lo, *a.shape[2:], dtype=a.dtype, device=a.device)
                _grad_a(dc, b, a_mn, b_mn, alpha, full)
                ga = full.reshape(a.shape[0], a.shape[1], n_lo // a.shape[1], *a.shape[2:]).float().sum(2).to(a.dtype)
            else:
                _grad_a(dc, b, a_mn, b_mn, alpha, ga)
            da = ga
        if ctx.needs_input_grad[1]:
            gb = _empty_like_layout(b) if b.shape[1] == n_lo else None
            if gb is None:
                full = torch.empty(b.shape[0], n_lo, *b.shape[2:], dtype=b.dtype, device=b.device)
                _grad_b(dc, a, a_mn, b_mn, alpha, full)
                gb = full.reshape(b.shape[0], b.shape[1], n_lo // b.shape[1], *b.shape[2:]).float().sum(2).to(b.dtype)
            else:
                _grad_b(dc, a, a_mn, b_mn, alpha, gb)
            db = gb
        return da, db, None, None, None, None, None, (dc if ctx.has_addend else None)


def _grad_a(dc, b, a_mn, b_mn, alpha, out):
    # dA[M,K] = dC[M,N] B[N,K]; B as the "N'=K" operand has its storage sense flipped
    if not a_mn:
        bgemm(dc, b, a_mn=False, b_mn=not b_mn, out=out, alpha=alpha)
    else:  # A stored [K, M]: dA^T[K,M] = B^T[K,N] dC^T[N,M]
        bgemm(b, dc, a_mn=not b_mn, b_mn=False, out=out, alpha=alpha)


def _grad_b(dc, a, a_mn, b_mn, alpha, out):
    # dB[N,K] = dC^T[N,M] A[M,K]
    if not b_mn:
        bgemm(dc, a, a_mn=True, b_mn=not a_mn, out=out, alpha=alpha)
    else:  # B stored [K, N]: dB^T[K,N] = A^T[K,M] dC[M,N]
        bgemm(a, dc, a_mn=not a_mn, b_mn=True, out=out, alpha=alpha)


def bmm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, alpha: float = 1.0,
        token_major: bool = False, out_dtype: Optional[torch.dtype] = None,
        addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable ``alpha * a @ b^T (+ addend)`` over ``[hi, lo, rows, inner]`` operands (see the module docstring).
    ``token_major`` stores the result as ``[hi, M, lo, N]`` (returned as the permuted view) so that a result whose
    rows are tokens lands in the chunk layout.  ``addend`` (shape and layout of the result) is added in the epilogue."""
    return _BMM.apply(a, b, a_mn, b_mn, alpha, token_major, out_dtype, addend)
