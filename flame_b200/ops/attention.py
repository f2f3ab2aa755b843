"""Variable-length causal softmax attention.

``attention(q, k, v, meta, scale, window)`` takes packed tensors ``q [T, H, Dh]``, ``k/v [T, Hkv, Dh]`` (any token
stride, so the three may be slices of one fused projection output) and the batch's ``VarlenMeta``.  On CUDA
it runs the tcgen05 kernels of ``csrc/attention.cu``; elsewhere it evaluates the plain softmax definition per
document in the input dtype, which is also the oracle of the kernel tests.

Counterpart of ``flash_attn_varlen_func`` as used by fla/layers/attn.py:146-174 (causal, optional sliding
window ``(window - 1, 0)``).
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib, sac
from .varlen import VarlenMeta

vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
_lib.register("fb_attn_fwd", [vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, i64, i64, i64, f32, i32, vp])
_lib.register("fb_attn_delta", [vp, vp, vp, i64, i32, i32, i64, i64, vp])
_lib.register("fb_attn_bwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, i32,
                              i64, i64, i64, i64, i64, i64, f32, i32, vp])


def attention_reference(q, k, v, meta: VarlenMeta, scale: float, window: int = 0) -> torch.Tensor:
    """Softmax attention per document, written out directly (O(L^2) memory per document)."""
    T, H, Dh = q.shape
    Hkv = k.shape[1]
    out = torch.empty(T, H, Dh, dtype=q.dtype, device=q.device)
    cu = meta.cu_cpu().tolist()
    rep = H // Hkv
    for a, b in zip(cu[:-1], cu[1:]):
        if b == a:
            continue
        qq = q[a:b].transpose(0, 1).float()
        kk = k[a:b].transpose(0, 1).float().repeat_interleave(rep, 0)
        vv = v[a:b].transpose(0, 1).float().repeat_interleave(rep, 0)
        L = b - a
        s = torch.matmul(qq, kk.transpose(1, 2)) * scale
        idx = torch.arange(L, device=q.device)
        mask = idx[None, :] > idx[:, None]
        if window and window > 0:
            mask = mask | (idx[None, :] <= idx[:, None] - window)
        s = s.masked_fill(mask[None], float("-inf"))
        o = torch.matmul(torch.softmax(s, -1), vv)
        out[a:b] = o.transpose(0, 1).to(q.dtype)
    return out


def _kernel_ok(q: torch.Tensor) -> bool:
    return _lib.available() and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta: VarlenMeta, scale: float, window: int, known=None):
        T, H, Dh = q.shape
        Hkv = k.shape[1]
        assert q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1
        assert q.stride(1) == Dh and k.stride(1) == Dh and v.stride(1) == Dh
        if known is not None:  # replay pass of operator-level selective checkpointing: output and lse are at hand
            o, lse = known
            ctx.save_for_backward(q, k, v, o, lse)
            ctx.meta, ctx.scale, ctx.window = meta, scale, window
            ctx.mark_non_differentiable(lse)
            return o.view_as(o), lse
        o = torch.empty(T, H, Dh, dtype=q.dtype, device=q.device)
        lse = torch.empty(H, T, dtype=torch.float32, device=q.device)
        rc = _lib.lib().fb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                    meta.cu_seqlens.data_ptr(), meta.tile_offsets.data_ptr(), meta.nseq,
                                    meta.max_tiles128, T, H, Hkv, Dh, q.stride(0), k.stride(0), v.stride(0),
                                    o.stride(0), float(scale), int(window), _lib.stream_ptr())
        _lib.check(rc, "fb_attn_fwd")
        _lib.count_launch()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta, ctx.scale, ctx.window = meta, scale, window
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse=None):
        q, k, v, o, lse = ctx.saved_tensors
        meta = ctx.meta
        T, H, Dh = q.shape
        Hkv = k.shape[1]
        do = do.contiguous()
        L = _lib.lib()
        delta = torch.empty(H, T, dtype=torch.float32, device=q.device)
        rc = L.fb_attn_delta(o.data_ptr(), do.data_ptr(), delta.data_ptr(), T, H, Dh, o.stride(0), do.stride(0),
                             _lib.stream_ptr())
        _lib.check(rc, "fb_attn_delta")
        dq_acc = torch.zeros(T, H, Dh, dtype=torch.float32, device=q.device)
        # dk/dv land in one fused buffer laid out like a qkv projection output: [T, (H + 2 Hkv) * Dh]
        dqkv = torch.empty(T, (H + 2 * Hkv) * Dh, dtype=q.dtype, device=q.device)
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
        dq.copy_(dq_acc)
        return dq, dk, dv, None, None, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: VarlenMeta, scale: Optional[float] = None,
              window: int = 0) -> torch.Tensor:
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if _kernel_ok(q):
        tape = sac.current() if torch.is_grad_enabled() else None
        if tape is not None and tape.mode == "record":
            tape.decide("attn")
            o, lse = _AttnFn.apply(q, k, v, meta, scale, window or 0, None)
            tape.store((o.detach(), lse))
            return o
        known = tape.fetch() if tape is not None else None
        return _AttnFn.apply(q, k, v, meta, scale, window or 0, known)[0]
    return attention_reference(q, k, v, meta, scale, window or 0)
