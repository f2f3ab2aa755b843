"""Rotary position embedding for packed sequences (NeoX half-split layout).

Positions restart at every document boundary, as in fla/modules/rotary.py:70-88; cos/sin come from an fp32
table indexed by the per-token position produced once per batch by ``VarlenMeta``.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from . import _lib

vp, i32, i64 = c_void_p, c_int, c_longlong
_lib.register("fb_rope", [vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i64, i32, i32, i32, vp])

_TABLES: dict = {}


def rope_tables(rot_dim: int, max_pos: int, base: float, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos, sin`` of shape ``[max_pos, rot_dim / 2]`` (cached per device)."""
    key = (rot_dim, float(base), str(device))
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < max_pos:
        n = max(max_pos, 2048)
        inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
        ang = torch.outer(torch.arange(n, dtype=torch.float32, device=device), inv)
        have = (ang.cos().contiguous(), ang.sin().contiguous())
        _TABLES[key] = have
    return have


def rope_reference(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   conj: bool = False) -> torch.Tensor:
    """x [T, H, Dh]; rotates the first ``2 * cos.shape[1]`` features of every head."""
    half = cos.shape[1]
    c = cos[pos.long()][:, None, :]
    s = sin[pos.long()][:, None, :]
    if conj:
        s = -s
    xf = x.float()
    x1, x2, rest = xf[..., :half], xf[..., half:2 * half], xf[..., 2 * half:]
    out = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, rest], dim=-1)
    return out.to(x.dtype)


def rope_inplace_(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, conj: bool = False) -> None:
    """In-place rotation of a ``[T, H, Dh]`` view (token stride arbitrary, head stride Dh)."""
    T, H, Dh = x.shape
    rot = 2 * cos.shape[1]
    if _lib.available() and x.is_cuda and x.dtype == torch.bfloat16 and rot % 16 == 0:
        assert x.stride(2) == 1 and x.stride(1) == Dh
        rc = _lib.lib().fb_rope(x.data_ptr(), x.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, H, Dh, rot,
                                x.stride(0), x.stride(0), 0, 1 if conj else 0, 0, _lib.stream_ptr())
        _lib.check(rc, "fb_rope")
        _lib.count_launch()
    else:
        x.copy_(rope_reference(x, pos, cos, sin, conj))


def rope_from_fp32_(src: torch.Tensor, dst: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                    conj: bool = False) -> None:
    """``dst (bf16 view) = rotate(src (fp32, contiguous [T, H, Dh]))``: the dtype conversion rides on the rotation."""
    T, H, Dh = src.shape
    rot = 2 * cos.shape[1]
    assert rot == Dh and src.dtype == torch.float32 and dst.dtype == torch.bfloat16
    rc = _lib.lib().fb_rope(src.data_ptr(), dst.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, H, Dh, rot,
                            src.stride(0), dst.stride(0), 0, 1 if conj else 0, 1, _lib.stream_ptr())
    _lib.check(rc, "fb_rope")
    _lib.count_launch()


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, cos, sin):
        y = x.contiguous().clone()
        rope_inplace_(y, pos, cos, sin, False)
        ctx.save_for_backward(pos, cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        pos, cos, sin = ctx.saved_tensors
        dx = dy.contiguous().clone()
        rope_inplace_(dx, pos, cos, sin, True)
        return dx, None, None, None


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Out-of-place, differentiable RoPE on ``[T, H, Dh]``."""
    return _RopeFn.apply(x, pos, cos, sin)
