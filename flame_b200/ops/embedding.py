"""Token embedding: gather forward, deterministic scatter-add backward.

The backward sorts the token ids once (stable), then one warp per distinct id sums that id's gradient rows in
sorted order and adds the total to the fp32 gradient row, so the result does not depend on atomics order
(ATen's embedding backward, used by the reference, accumulates with atomics).
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p

import torch
import torch.nn.functional as F

from . import _lib

vp, i32, i64 = c_void_p, c_int, c_longlong
_lib.register("fb_embedding_fwd", [vp, vp, vp, i64, i32, i64, vp])
_lib.register("fb_embedding_bwd_sorted", [vp, vp, vp, i32, i64, vp, vp, i32, i64, vp])


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        shape = ids.shape
        flat = ids.reshape(-1).contiguous()
        T = flat.numel()
        V, D = weight.shape
        out = torch.empty(T, D, dtype=weight.dtype, device=weight.device)
        rc = _lib.lib().fb_embedding_fwd(flat.data_ptr(), weight.data_ptr(), out.data_ptr(), T, D, V, _lib.stream_ptr())
        _lib.check(rc, "fb_embedding_fwd")
        _lib.count_launch()
        ctx.save_for_backward(flat, weight)
        return out.view(*shape, D)

    @staticmethod
    def backward(ctx, dout):
        flat, weight = ctx.saved_tensors
        V, D = weight.shape
        T = flat.numel()
        d2 = dout.reshape(T, D)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        sorted_ids, perm = torch.sort(flat, stable=True)
        is_start = torch.ones(T, dtype=torch.bool, device=flat.device)
        is_start[1:] = sorted_ids[1:] != sorted_ids[:-1]
        seg_start = torch.nonzero(is_start).flatten().to(torch.int32)
        nseg = seg_start.numel()
        mg = getattr(weight, "main_grad", None)
        dtable = mg if mg is not None else torch.zeros(V, D, dtype=torch.float32, device=weight.device)
        rc = _lib.lib().fb_embedding_bwd_sorted(sorted_ids.data_ptr(), perm.data_ptr(), seg_start.data_ptr(), nseg, T,
                                                d2.data_ptr(), dtable.data_ptr(), D, V, _lib.stream_ptr())
        _lib.check(rc, "fb_embedding_bwd_sorted")
        _lib.count_launch()
        return None, (None if mg is not None else dtable.to(weight.dtype))


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if _lib.available() and weight.is_cuda and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, weight)
    return F.embedding(ids, weight)
