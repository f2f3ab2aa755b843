"""Stick-breaking attention: ``sb_attention(q, k, v, meta) -> (out, remainder)``.

``att_ij = sigmoid(l_ij) * prod_{j<m<i} (1 - sigmoid(l_im))`` for ``j < i`` inside one document, ``out = att @ v``,
``remainder = 1 - sum_j att_ij``.  On CUDA (bf16, head dim 64) the tcgen05 kernels of ``csrc/attention.cu`` (forward)
and ``csrc/sb_attention.cu`` (backward) run; packed documents are supported, which the reference layer does not offer
(custom_models/sba/sba_layer.py:84-87 asserts ``cu_seqlens is None``).  Elsewhere the definition is evaluated directly.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from . import _lib, linear_attn as la
from .varlen import VarlenMeta

vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
_lib.register("fb_sb_attn_fwd", [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, i64, i64, i64, i64, f32, vp])
_lib.register("fb_sb_attn_bwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32,
                                 i64, i64, i64, i64, i64, i64, f32, vp])


class _SBFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta: VarlenMeta, scale: float):
        T, H, Dh = q.shape
        o = torch.empty(T, H, Dh, dtype=q.dtype, device=q.device)
        # the low half of a two-term bf16 split of the fp32 output: the backward's prefix sums need do . o to fp32 accuracy
        o_lo = torch.empty(T, H, Dh, dtype=q.dtype, device=q.device) if any(ctx.needs_input_grad[:3]) else None
        rem = torch.ones(H, T, dtype=torch.float32, device=q.device)
        rc = _lib.lib().fb_sb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), _lib.ptr(o_lo), rem.data_ptr(),
                                       meta.cu_seqlens.data_ptr(), meta.tile_offsets.data_ptr(), meta.nseq,
                                       meta.max_tiles128, T, H, Dh, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
                                       float(scale), _lib.stream_ptr())
        _lib.check(rc, "fb_sb_attn_fwd")
        _lib.count_launch()
        ctx.save_for_backward(q, k, v, o, rem, o_lo)
        ctx.meta, ctx.scale = meta, scale
        return o, rem.t()

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, o, rem, o_lo = ctx.saved_tensors
        meta = ctx.meta
        T, H, Dh = q.shape
        do = do if do.is_contiguous() else do.contiguous()
        dr = None
        if drem is not None and ctx.needs_input_grad[0]:
            dr = drem.t().contiguous().float()
        dev = q.device
        tot = torch.empty(H, T, dtype=torch.float32, device=dev)
        dq = torch.empty(T, H, Dh, dtype=q.dtype, device=dev)
        dkv = torch.zeros(2, T, H, Dh, dtype=torch.float32, device=dev)
        rc = _lib.lib().fb_sb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), _lib.ptr(o_lo), do.data_ptr(),
                                       rem.data_ptr(), _lib.ptr(dr), tot.data_ptr(), dq.data_ptr(), dkv[0].data_ptr(),
                                       dkv[1].data_ptr(), meta.cu_seqlens.data_ptr(), meta.tile_offsets.data_ptr(),
                                       meta.nseq, meta.max_tiles128, T, H, q.stride(0), k.stride(0), v.stride(0),
                                       o.stride(0), do.stride(0), dq.stride(0), float(ctx.scale), _lib.stream_ptr())
        _lib.check(rc, "fb_sb_attn_bwd")
        _lib.count_launch(2)
        return dq, dkv[0].to(q.dtype), dkv[1].to(q.dtype), None, None


def sb_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: VarlenMeta,
                 scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k, v ``[T, H, Dh]`` (head stride Dh, any token stride) -> (``[T, H, Dh]``, remainder ``[T, H]``)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:   # context parallelism cut the row inside documents: borrow the first document's earlier rows
        from ..parallel.context_parallel import borrow_prefix
        q, k, v = borrow_prefix([q, k, v], sl)
        o, rem = sb_attention(q, k, v, sl.ext_meta, scale)
        return o[sl.prefix:], rem[sl.prefix:]
    if (_lib.available() and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 64 and q.stride(1) == 64
            and k.stride(1) == 64 and v.stride(1) == 64 and q.stride(2) == 1):
        return _SBFn.apply(q, k, v, meta, scale)
    return la.stickbreaking_reference(q, k, v, meta, scale)
