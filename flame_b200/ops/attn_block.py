"""Fused "RoPE + varlen attention" node working directly on a fused qkv projection output.

Input is the ``[T, (H + 2 Hkv) * Dh]`` output of one qkv GEMM.  RoPE is applied in place on the q and k column
blocks, attention reads q/k/v as strided views of that same buffer, and the backward produces a single
``[T, (H + 2 Hkv) * Dh]`` gradient buffer (inverse RoPE applied in place) that feeds ONE weight-gradient GEMM.
The reference does these as separate kernels on separate tensors (fla/layers/attn.py:102-176).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .attention import _AttnFn, _kernel_ok, attention_reference
from .rope import rope_from_fp32_, rope_inplace_, rope_reference
from .varlen import VarlenMeta


class _QkvAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, meta: VarlenMeta, H, Hkv, Dh, cos, sin, scale, window):
        T = qkv.shape[0]
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        q = qkv[:, : H * Dh].view(T, H, Dh)
        k = qkv[:, H * Dh: (H + Hkv) * Dh].view(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        if cos is not None:
            # q and k are adjacent column blocks of the fused buffer: one launch rotates both
            qk = qkv[:, : (H + Hkv) * Dh].view(T, H + Hkv, Dh)
            rope_inplace_(qk, meta.position_ids, cos, sin)
        L = _lib.lib()
        o = torch.empty(T, H, Dh, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(H, T, dtype=torch.float32, device=qkv.device)
        rc = L.fb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                           meta.cu_seqlens.data_ptr(), meta.tile_offsets.data_ptr(), meta.nseq, meta.max_tiles128, T, H,
                           Hkv, Dh, q.stride(0), k.stride(0), v.stride(0), o.stride(0), float(scale), int(window),
                           _lib.stream_ptr())
        _lib.check(rc, "fb_attn_fwd")
        _lib.count_launch()
        ctx.save_for_backward(qkv, o, lse, cos, sin)
        ctx.meta, ctx.dims, ctx.scale, ctx.window = meta, (H, Hkv, Dh), scale, window
        return o.view(T, H * Dh)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin = ctx.saved_tensors
        meta = ctx.meta
        H, Hkv, Dh = ctx.dims
        T = qkv.shape[0]
        q = qkv[:, : H * Dh].view(T, H, Dh)
        k = qkv[:, H * Dh: (H + Hkv) * Dh].view(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        do = do.reshape(T, H, Dh)
        do = do if do.is_contiguous() else do.contiguous()
        L = _lib.lib()
        delta = torch.empty(H, T, dtype=torch.float32, device=qkv.device)
        rc = L.fb_attn_delta(o.data_ptr(), do.data_ptr(), delta.data_ptr(), T, H, Dh, o.stride(0), do.stride(0),
                             _lib.stream_ptr())
        _lib.check(rc, "fb_attn_delta")
        dq_acc = torch.zeros(T, H, Dh, dtype=torch.float32, device=qkv.device)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, : H * Dh].view(T, H, Dh)
        dk = dqkv[:, H * Dh: (H + Hkv) * Dh].view(T, Hkv, Dh)
        dv = dqkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        rc = L.fb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                           dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), meta.cu_seqlens.data_ptr(),
                           meta.tile_offsets.data_ptr(), meta.nseq, meta.max_tiles128, T, H, Hkv, Dh, q.stride(0),
                           k.stride(0), v.stride(0), do.stride(0), dk.stride(0), dv.stride(0), float(ctx.scale),
                           int(ctx.window), _lib.stream_ptr())
        _lib.check(rc, "fb_attn_bwd")
        _lib.count_launch(2)
        if cos is not None and 2 * cos.shape[1] == Dh:
            pos = meta.position_ids
            rope_from_fp32_(dq_acc, dq, pos, cos, sin, conj=True)  # fp32 -> bf16 conversion fused with the rotation
            rope_inplace_(dk, pos, cos, sin, conj=True)
        else:
            dq.copy_(dq_acc)
            if cos is not None:
                pos = meta.position_ids
                rope_inplace_(dq, pos, cos, sin, conj=True)
                rope_inplace_(dk, pos, cos, sin, conj=True)
        return dqkv, None, None, None, None, None, None, None, None


def qkv_attention(qkv: torch.Tensor, meta: VarlenMeta, H: int, Hkv: int, Dh: int,
                  rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, scale: Optional[float] = None,
                  window: int = 0) -> torch.Tensor:
    """Returns the attention output ``[T, H * Dh]`` for a fused qkv buffer ``[T, (H + 2 Hkv) * Dh]``."""
    if scale is None:
        scale = 1.0 / math.sqrt(Dh)
    cos, sin = rope if rope is not None else (None, None)
    T = qkv.shape[0]
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:
        # context parallelism that cut the row inside documents: this rank's queries, everybody's keys and values
        from ..parallel.context_parallel import sequence_parallel_attention
        q = qkv[:, : H * Dh].reshape(T, H, Dh)
        k = qkv[:, H * Dh: (H + Hkv) * Dh].reshape(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].reshape(T, Hkv, Dh)
        if cos is not None:
            pos = meta.position_ids
            if _lib.available() and qkv.is_cuda and qkv.dtype == torch.bfloat16:
                from .rope import apply_rope
                q, k = apply_rope(q, pos, cos, sin), apply_rope(k, pos, cos, sin)
            else:
                q, k = rope_reference(q, pos, cos, sin), rope_reference(k, pos, cos, sin)
        return sequence_parallel_attention(q, k, v, sl, scale, window or 0).reshape(T, H * Dh)
    if _lib.available() and qkv.is_cuda and qkv.dtype == torch.bfloat16 and Dh == 64:
        return _QkvAttnFn.apply(qkv, meta, H, Hkv, Dh, cos, sin, scale, window or 0)
    q = qkv[:, : H * Dh].reshape(T, H, Dh)
    k = qkv[:, H * Dh: (H + Hkv) * Dh].reshape(T, Hkv, Dh)
    v = qkv[:, (H + Hkv) * Dh:].reshape(T, Hkv, Dh)
    if cos is not None:
        pos = meta.position_ids
        if _lib.available() and qkv.is_cuda and qkv.dtype == torch.bfloat16:
            from .rope import apply_rope
            q, k = apply_rope(q, pos, cos, sin), apply_rope(k, pos, cos, sin)
        else:
            q, k = rope_reference(q, pos, cos, sin), rope_reference(k, pos, cos, sin)
    from .attention import attention
    return attention(q.contiguous(), k.contiguous(), v.contiguous(), meta, scale, window or 0).reshape(T, H * Dh)
