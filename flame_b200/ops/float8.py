"""Float8 training for linear layers: tensor-wise dynamic scaling on the fp8 tcgen05 GEMM.

``--model.converters float8`` in the reference swaps every ``nn.Linear`` for torchao's ``Float8Linear``
(torchtitan/components/quantization/float8.py:30-137, "tensorwise" recipe): activations and weights are
cast to e4m3 and output gradients to e5m2, each with one scale per tensor computed from the tensor's current
absolute maximum, and all three products of the layer (output, input gradient, weight gradient) run as fp8
GEMMs with fp32 accumulation.  Here the same arithmetic is

* ``quantize(x)``: ``csrc/fp8.cu`` -- amax, cast, and the transposed 8-bit copy the backward products read
  (the GEMM takes both operands K-major), plus the dequantisation factor as a device scalar;
* ``gemm_fp8(a, b)``: ``csrc/gemm2.cu`` with ``kind::f8f6f4`` MMAs, the two dequantisation factors read from
  device memory and folded into the epilogue (no host synchronisation anywhere).

Weights opt in by carrying ``_fp8 = True`` (set by ``convert_to_float8``); ``ops.linear`` routes such
weights through ``float8_linear_forward`` / ``float8_linear_backward``.  Without CUDA the same functions
compute with torch's float8 dtypes, which is what the CPU tests check the kernels against.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Iterable, Optional, Tuple

import torch

from . import _lib

E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2
_FMAX = {E4M3: 448.0, E5M2: 57344.0}

_lib.register("fb_fp8_quantize", [c_void_p, c_longlong, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p])
_lib.register("fb_gemm2_fp8", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                               c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])

_SM_COUNT: dict = {}


def _sm_count(device: torch.device) -> int:
    n = _SM_COUNT.get(device.index)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _SM_COUNT[device.index] = n
    return n


def supported(x: torch.Tensor) -> bool:
    """Shapes the kernels take: a bf16 matrix whose two extents are multiples of 16."""
    return x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[0] % 16 == 0 and x.shape[1] % 16 == 0


def quantize(x: torch.Tensor, dtype: torch.dtype = E4M3, transpose: bool = True
             ) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """``x [R, C]`` -> ``(q [R, C], qT [C, R] or None, inv_scale [1] fp32)`` with ``x ~= q * inv_scale``."""
    R, C = x.shape
    fmax = _FMAX[dtype]
    if _lib.available() and x.is_cuda:
        if not supported(x):
            raise ValueError(f"float8 quantisation needs a bf16 matrix with extents that are multiples of 16, got "
                             f"{tuple(x.shape)} {x.dtype}")
        if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
            x = x.contiguous()
        q = torch.empty(R, C, dtype=dtype, device=x.device)
        qT = torch.empty(C, R, dtype=dtype, device=x.device) if transpose else None
        scal = torch.empty(2, dtype=torch.float32, device=x.device)  # [amax scratch, inv_scale]
        rc = _lib.lib().fb_fp8_quantize(x.data_ptr(), R, C, x.stride(0), int(dtype == E5M2), q.data_ptr(),
                                        _lib.ptr(qT), scal.data_ptr(), scal.data_ptr() + 4, _lib.stream_ptr())
        _lib.check(rc, "fb_fp8_quantize")
        _lib.count_launch(2)
        return q, qT, scal[1:2]
    amax = x.detach().abs().max().float().clamp_min(1e-12)
    scaled = (x.detach().float() * (fmax / amax)).clamp(-fmax, fmax)
    q = scaled.to(dtype)
    qT = q.t().contiguous() if transpose else None
    return q, qT, (amax / fmax).reshape(1)


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, inv_a: torch.Tensor, inv_b: torch.Tensor,
             out: Optional[torch.Tensor] = None, *, out_dtype: torch.dtype = torch.bfloat16,
             accumulate: bool = False) -> torch.Tensor:
    """``(a [M, K] * inv_a) @ (b [N, K] * inv_b).T`` with 8-bit ``a``, ``b``; bf16 or fp32 (optionally accumulated) out."""
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape)
    if _lib.available() and a.is_cuda:
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype, device=a.device)
        if out.dtype == torch.bfloat16:
            if accumulate:
                raise ValueError("accumulation needs an fp32 output")
            mode = 0
        elif out.dtype == torch.float32:
            mode = 2 if accumulate else 1
        else:
            raise ValueError(f"unsupported output dtype {out.dtype}")
        if out.stride(-1) != 1 or not a.is_contiguous() or not b.is_contiguous() or K % 16:
            raise ValueError("fp8 GEMM operands must be contiguous with K a multiple of 16, the output row-major")
        rc = _lib.lib().fb_gemm2_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, K, K, out.stride(0),
                                     int(a.dtype == E5M2), int(b.dtype == E5M2), inv_a.data_ptr(), inv_b.data_ptr(),
                                     mode, 1.0, _sm_count(a.device), _lib.stream_ptr())
        _lib.check(rc, "fb_gemm2_fp8")
        _lib.count_launch(1)
        return out
    r = (a.float() @ b.float().t()) * (inv_a.float() * inv_b.float())
    if out is None:
        return r.to(out_dtype)
    if accumulate:
        out += r.to(out.dtype)
    else:
        out.copy_(r)
    return out


ROWWISE = ("rowwise", "rowwise_with_gw_hp")


def quantize_rows(x: torch.Tensor, dtype: torch.dtype = E4M3) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per row, rounded down to a power of two (the row-wise recipes of the reference's converter,
    torchtitan/components/quantization/float8.py:52-64 with torchao's ``Float8LinearConfig.from_recipe_name``):
    ``x [R, C]`` -> ``(q [R, C] 8-bit, inv_scale [R] fp32)`` with ``x ~= q * inv_scale[:, None]``."""
    fmax = _FMAX[dtype]
    amax = x.detach().abs().amax(dim=1).float().clamp_min(1e-12)
    scale = torch.exp2(torch.floor(torch.log2(fmax / amax)))
    q = (x.detach().float() * scale[:, None]).clamp(-fmax, fmax).to(dtype)
    return q, 1.0 / scale


def gemm_fp8_rows(a: torch.Tensor, a_inv: torch.Tensor, b: torch.Tensor, b_inv: torch.Tensor) -> torch.Tensor:
    """``(a * a_inv[:, None]) @ (b * b_inv[:, None]).T`` in fp32 for row-scaled 8-bit operands: the fp8 GEMM with unit
    factors, then the outer product of the two scale vectors (the GEMM's epilogue takes one factor per operand, so the
    per-row factors are applied to its fp32 result)."""
    if _lib.available() and a.is_cuda and a.shape[1] % 16 == 0 and a.shape[0] % 16 == 0 and b.shape[0] % 16 == 0:
        one = torch.ones(1, dtype=torch.float32, device=a.device)
        r = gemm_fp8(a.contiguous(), b.contiguous(), one, one, out_dtype=torch.float32)
    else:
        r = a.float() @ b.float().t()
    return r.mul_(a_inv[:, None]).mul_(b_inv[None, :])


def float8_linear_forward(x2: torch.Tensor, w: torch.Tensor, recipe="tensorwise"):
    """``y = x2 @ w.T`` in fp8; returns ``(y, saved)`` where ``saved`` holds what the backward needs.  Tensor-wise: the
    transposed 8-bit copies of input and weight and their factors (the bf16 input itself is not kept).  Row-wise: the
    input and the weight themselves, because every product of the backward scales them along a different axis."""
    if recipe in ROWWISE:
        xq, x_inv = quantize_rows(x2, E4M3)     # one scale per token
        wq, w_inv = quantize_rows(w, E4M3)      # one scale per output feature
        return gemm_fp8_rows(xq, x_inv, wq, w_inv).to(x2.dtype), (x2, w)
    xq, xqT, x_inv = quantize(x2, E4M3, transpose=True)
    wq, wqT, w_inv = quantize(w, E4M3, transpose=True)
    y = gemm_fp8(xq, wq, x_inv, w_inv, out_dtype=x2.dtype)
    return y, (xqT, x_inv, wqT, w_inv)


def float8_linear_backward(dy2: torch.Tensor, saved, need_dx: bool, wgrad_out: Optional[torch.Tensor] = None,
                           need_dw: bool = True, recipe="tensorwise"):
    """Returns ``(dx or None, dw or None)``; with ``wgrad_out`` (fp32 [N, K]) the weight gradient is accumulated there
    and ``dw`` is None."""
    if recipe in ROWWISE:
        x2, w = saved
        dx = None
        if need_dx:
            dq, d_inv = quantize_rows(dy2, E5M2)                      # per token
            wtq, wt_inv = quantize_rows(w.t().contiguous(), E4M3)     # per input feature
            dx = gemm_fp8_rows(dq, d_inv, wtq, wt_inv).to(dy2.dtype)
        dw = None
        if need_dw:
            if recipe == "rowwise_with_gw_hp":
                # the weight-gradient product stays in bf16 (the tcgen05 GEMM with fp32 accumulation on the GPU)
                if _lib.available() and dy2.is_cuda and dy2.dtype == torch.bfloat16:
                    from .gemm import gemm_tn
                    dw = gemm_tn(dy2.contiguous(), x2.contiguous(), out_dtype=torch.float32)
                else:
                    dw = dy2.float().t() @ x2.float()
            else:
                dtq, dt_inv = quantize_rows(dy2.t().contiguous(), E5M2)   # per output feature, over the tokens
                xtq, xt_inv = quantize_rows(x2.t().contiguous(), E4M3)    # per input feature, over the tokens
                dw = gemm_fp8_rows(dtq, dt_inv, xtq, xt_inv)
            if wgrad_out is not None:
                wgrad_out += dw
                dw = None
        return dx, dw
    xqT, x_inv, wqT, w_inv = saved
    dq, dqT, d_inv = quantize(dy2, E5M2, transpose=need_dw)
    dx = gemm_fp8(dq, wqT, d_inv, w_inv, out_dtype=dy2.dtype) if need_dx else None
    dw = None
    if need_dw:
        if wgrad_out is not None:
            gemm_fp8(dqT, xqT, d_inv, x_inv, out=wgrad_out, accumulate=True)
        else:
            dw = gemm_fp8(dqT, xqT, d_inv, x_inv, out_dtype=torch.float32)
    return dx, dw


def convert_to_float8(model: torch.nn.Module, filter_fqns: Iterable[str] = ("lm_head",), recipe: Optional[str] = None,
                      min_dim: int = 0) -> int:
    """Marks the weights of the model's linear projections for fp8 execution and returns how many were marked.

    The rule follows the reference's converter: 2-D projection weights whose extents are multiples of 16, except
    modules whose qualified name contains one of ``filter_fqns`` (the output head by default), embeddings and
    normalisation weights.  ``min_dim`` leaves out projections with a smaller extent than that (low-rank gate
    projections and the like, where the casts cost more than the GEMM saves).  ``recipe``: ``tensorwise`` (the fused cast
    kernels and scalar factors in the GEMM epilogue), ``rowwise`` / ``rowwise_with_gw_hp`` (one power-of-two scale per row
    of every operand, applied to the GEMM's fp32 result; the second keeps the weight-gradient product in bf16).
    """
    recipe = recipe or "tensorwise"
    if recipe not in ("tensorwise",) + ROWWISE:
        raise ValueError(f"unknown float8 recipe {recipe!r}")
    skip = tuple(filter_fqns)
    n = 0
    for name, p in model.named_parameters():
        if p.dim() != 2 or not name.endswith("weight"):
            continue
        if any(s in name for s in skip) or "embed" in name or "norm" in name or "conv" in name:
            continue
        if p.shape[0] % 16 or p.shape[1] % 16 or min(p.shape) < min_dim:
            continue
        p._fp8 = recipe   # truthy: the recipe's name
        n += 1
    return n
