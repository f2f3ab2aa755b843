"""Fused gate arithmetic of the linear-attention layers (one kernel pass each way instead of a chain of elementwise
framework kernels).

``hgrn2_gates(q_raw, f_raw, lower_bound)`` returns ``(q, k, g)`` of fla/layers/hgrn2.py:160-190:
``q = silu(q_raw)``, ``g = logsigmoid(f_raw)`` (with a lower bound: ``g = log(lb + (1 - lb) sigmoid(f_raw))``, the closed
form of the reference's ``logaddexp(log lb, log1p(-lb) + logsigmoid f)``), ``k = 1 - exp(g)``; ``g`` in fp32.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

_lib.register("fb_hgrn2_gate_tiles", [c_longlong])
_lib.register("fb_hgrn2_gate_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
_lib.register("fb_hgrn2_gate_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_longlong, c_int, c_void_p])


def hgrn2_gates_reference(q_raw: torch.Tensor, f_raw: torch.Tensor,
                          lower_bound: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    q = F.silu(q_raw)
    g = F.logsigmoid(f_raw.float())
    if lower_bound is not None:
        lb = lower_bound.float()
        g = torch.logaddexp(lb.log(), torch.log1p(-lb) + g)
    k = (1 - g.exp()).to(q_raw.dtype)
    return q, k, g


class _Hgrn2Gates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_raw, f_raw, lb):
        rows, D = q_raw.shape
        q_raw, f_raw = q_raw.contiguous(), f_raw.contiguous()
        lbf = lb.detach().float().contiguous() if lb is not None else None
        q, k = torch.empty_like(q_raw), torch.empty_like(q_raw)
        g = torch.empty(rows, D, dtype=torch.float32, device=q_raw.device)
        rc = _lib.lib().fb_hgrn2_gate_fwd(q_raw.data_ptr(), f_raw.data_ptr(), _lib.ptr(lbf), q.data_ptr(), k.data_ptr(),
                                          g.data_ptr(), rows, D, _lib.stream_ptr())
        _lib.check(rc, "fb_hgrn2_gate_fwd")
        _lib.count_launch()
        ctx.save_for_backward(q_raw, f_raw, lbf)
        ctx.lb_dtype = lb.dtype if lb is not None else None
        return q, k, g

    @staticmethod
    def backward(ctx, dq, dk, dg):
        q_raw, f_raw, lbf = ctx.saved_tensors
        rows, D = q_raw.shape
        L = _lib.lib()
        dq = torch.zeros_like(q_raw) if dq is None else dq.contiguous()
        dk = torch.zeros_like(q_raw) if dk is None else dk.contiguous()
        dg = torch.zeros(rows, D, dtype=torch.float32, device=q_raw.device) if dg is None else dg.float().contiguous()
        dq_raw, df_raw = torch.empty_like(q_raw), torch.empty_like(f_raw)
        part = dlb = None
        if lbf is not None:
            part = torch.empty(int(L.fb_hgrn2_gate_tiles(rows)), D, dtype=torch.float32, device=q_raw.device)
            dlb = torch.empty(D, dtype=torch.float32, device=q_raw.device)
        rc = L.fb_hgrn2_gate_bwd(q_raw.data_ptr(), f_raw.data_ptr(), _lib.ptr(lbf), dq.data_ptr(), dk.data_ptr(), dg.data_ptr(),
                                 dq_raw.data_ptr(), df_raw.data_ptr(), _lib.ptr(part), _lib.ptr(dlb), rows, D, _lib.stream_ptr())
        _lib.check(rc, "fb_hgrn2_gate_bwd")
        _lib.count_launch(2 if lbf is not None else 1)
        return dq_raw, df_raw, (dlb.to(ctx.lb_dtype) if dlb is not None else None)


def hgrn2_gates(q_raw: torch.Tensor, f_raw: torch.Tensor,
                lower_bound: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[T, D]`` bf16 projections (and an optional ``[D]`` lower bound) -> ``q`` bf16, ``k`` bf16, ``g`` fp32, all ``[T, D]``."""
    if (_lib.available() and q_raw.is_cuda and q_raw.dtype == torch.bfloat16 and f_raw.dtype == torch.bfloat16
            and q_raw.dim() == 2 and q_raw.shape == f_raw.shape and q_raw.shape[1] % 8 == 0):
        return _Hgrn2Gates.apply(q_raw, f_raw, lower_bound)
    return hgrn2_gates_reference(q_raw, f_raw, lower_bound)
