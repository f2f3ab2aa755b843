"""Linear layers on the tcgen05 GEMM, with the Megatron-style "main_grad" contract.

If a weight carries a ``main_grad`` attribute (an fp32 view into the sharding engine's flat gradient buffer)
the weight-gradient GEMM accumulates straight into it and autograd sees ``None`` for that weight; otherwise
the gradient is returned to autograd as usual.

``linear_fused(x, [w_q, w_k, w_v])`` runs ONE GEMM when the weights (and their ``main_grad``s) sit back to back
in memory, which is how the engine lays out a block's parameters; the HF-style per-projection parameter names
are kept for checkpoints (fla/layers/attn.py:73-82, fla/modules/mlp.py:58-60 use separate nn.Linear calls).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib, float8, sac
from .gemm import gemm_nn, gemm_nt, gemm_tn


def _adjacent(ts: Sequence[torch.Tensor]) -> bool:
    for a, b in zip(ts[:-1], ts[1:]):
        if not (a.is_contiguous() and b.is_contiguous()):
            return False
        if a.dtype != b.dtype or a.shape[1:] != b.shape[1:]:
            return False
        if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
            return False
        if a.storage_offset() + a.numel() != b.storage_offset():
            return False
    return True


def _cat_view(ts: Sequence[torch.Tensor]) -> torch.Tensor:
    first = ts[0]
    rows = sum(t.shape[0] for t in ts)
    out = torch.empty(0, dtype=first.dtype, device=first.device)
    out.set_(first.untyped_storage(), first.storage_offset(), (rows, *first.shape[1:]), first.stride())
    return out


def _kernel_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (_lib.available() and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0)


class _LinearFn(torch.autograd.Function):
    """y = x @ cat(weights).T (+ bias); weights are passed individually so autograd can route their grads."""

    @staticmethod
    def forward(ctx, x, bias, known, *weights):
        """``known``: the output when it is already at hand (the replay pass of operator-level selective activation
        checkpointing, ``ops/sac.py``): nothing is computed, the node only saves what its backward needs."""
        shape = x.shape
        K = shape[-1]
        x2 = x.reshape(-1, K)
        fused = len(weights) == 1 or _adjacent([w.detach() for w in weights])
        ctx.fp8 = (known is None and fused and bias is None and all(getattr(w, "_fp8", False) for w in weights)
                   and float8.supported(x2) and all(w.shape[0] % 16 == 0 for w in weights))
        # the parameters themselves (not the saved copies): under activation checkpointing the tensors that come back
        # from ``saved_tensors`` are detached recomputations without the ``main_grad`` attribute
        ctx.params = weights
        if known is not None:
            ctx.save_for_backward(x2, *weights)
            ctx.fused, ctx.shape, ctx.has_bias = fused, shape, bias is not None
            return known.view(*shape[:-1], known.shape[-1])
        if ctx.fp8:
            wcat = weights[0].detach() if len(weights) == 1 else _cat_view([w.detach() for w in weights])
            recipe = getattr(weights[0], "_fp8", None)
            ctx.fp8_recipe = recipe if isinstance(recipe, str) else "tensorwise"
            y, saved = float8.float8_linear_forward(x2, wcat, ctx.fp8_recipe)
            ctx.n_fp8_saved = len(saved)
            ctx.save_for_backward(*saved, *weights)
            ctx.fused, ctx.shape, ctx.has_bias = fused, shape, False
            return y.view(*shape[:-1], y.shape[-1])
        if fused:
            wcat = weights[0].detach() if len(weights) == 1 else _cat_view([w.detach() for w in weights])
            y = gemm_nt(x2, wcat, bias=bias)
        else:
            N = sum(w.shape[0] for w in weights)
            y = torch.empty(x2.shape[0], N, dtype=x.dtype, device=x.device)
            c = 0
            for w in weights:
                gemm_nt(x2, w.detach(), out=y[:, c:c + w.shape[0]])
                c += w.shape[0]
            if bias is not None:
                y += bias
        ctx.save_for_backward(x2, *weights)
        ctx.fused, ctx.shape, ctx.has_bias = fused, shape, bias is not None
        return y.view(*shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        if ctx.fp8:
            return _LinearFn._backward_fp8(ctx, dy)
        x2, *weights = ctx.saved_tensors
        N = dy.shape[-1]
        dy2 = dy.reshape(-1, N)
        if dy2.stride(-1) != 1 or dy2.stride(0) % 8 != 0:
            dy2 = dy2.contiguous()
        K = x2.shape[1]
        dx = None
        if ctx.needs_input_grad[0]:
            if ctx.fused:
                wcat = weights[0] if len(weights) == 1 else _cat_view(list(weights))
                dx = gemm_nn(dy2, wcat)
            else:
                dx32 = None
                c = 0
                for w in weights:
                    part = gemm_nn(dy2[:, c:c + w.shape[0]], w, out_dtype=torch.float32)
                    dx32 = part if dx32 is None else dx32.add_(part)
                    c += w.shape[0]
                dx = dx32.to(x2.dtype)
            dx = dx.view(ctx.shape)
        grads = [None] * len(weights)
        mgs = [getattr(w, "main_grad", None) for w in ctx.params]
        if all(m is not None for m in mgs):
            if ctx.fused and (len(weights) == 1 or _adjacent(mgs)):
                mg = mgs[0] if len(weights) == 1 else _cat_view(mgs)
                gemm_tn(dy2, x2, out=mg, accumulate=True)
            else:
                c = 0
                for w, m in zip(weights, mgs):
                    gemm_tn(dy2[:, c:c + w.shape[0]], x2, out=m, accumulate=True)
                    c += w.shape[0]
        else:
            c = 0
            for i, w in enumerate(weights):
                if ctx.needs_input_grad[3 + i]:
                    grads[i] = gemm_tn(dy2[:, c:c + w.shape[0]], x2, out_dtype=torch.float32).to(w.dtype)
                c += w.shape[0]
        gb = None
        if ctx.has_bias and ctx.needs_input_grad[1]:
            gb = dy2.float().sum(0).to(dy.dtype)
        return (dx, gb, None, *grads)


def _backward_fp8(ctx, dy):
    saved = tuple(ctx.saved_tensors[:ctx.n_fp8_saved])
    weights = list(ctx.saved_tensors[ctx.n_fp8_saved:])
    recipe = ctx.fp8_recipe
    dy2 = dy.reshape(-1, dy.shape[-1])
    need_dx = ctx.needs_input_grad[0]
    mgs = [getattr(w, "main_grad", None) for w in ctx.params]
    grads = [None] * len(weights)
    if all(m is not None for m in mgs) and (len(weights) == 1 or _adjacent(mgs)):
        mg = mgs[0] if len(weights) == 1 else _cat_view(mgs)
        dx, _ = float8.float8_linear_backward(dy2, saved, need_dx, wgrad_out=mg, recipe=recipe)
    else:
        need_dw = any(ctx.needs_input_grad[3:])
        dx, dw = float8.float8_linear_backward(dy2, saved, need_dx, need_dw=need_dw, recipe=recipe)
        c = 0
        for i, (w, m) in enumerate(zip(weights, mgs)):
            if dw is not None:
                part = dw[c:c + w.shape[0]]
                if m is not None:
                    m += part
                elif ctx.needs_input_grad[3 + i]:
                    grads[i] = part.to(w.dtype)
            c += w.shape[0]
    if dx is not None:
        dx = dx.view(ctx.shape)
    return (dx, None, None, *grads)


_LinearFn._backward_fp8 = staticmethod(_backward_fp8)


def _cpu_fp8(x: torch.Tensor, weights: Sequence[torch.Tensor]) -> bool:
    # without CUDA the fp8 path still runs (torch float8 dtypes) so that converted models behave the same everywhere
    return (all(getattr(w, "_fp8", False) for w in weights) and x.shape[-1] % 16 == 0
            and x.numel() // x.shape[-1] % 16 == 0)


def _with_tape(x: torch.Tensor, bias, weights: Sequence[torch.Tensor], compute):
    """Runs ``compute()`` unless a selective-checkpointing tape is active (``ops/sac.py``).  Under a tape both passes go
    through ``_LinearFn`` - with the output computed in the record pass and handed over in the replay pass - because the
    checkpoint machinery requires the recomputation to save the same tensors, in the same order, as the forward."""
    tape = sac.current()
    if tape is None or not torch.is_grad_enabled() or any(getattr(w, "_fp8", False) for w in weights):
        return compute()
    if tape.mode == "record":
        tape.decide("mm")
        y = _LinearFn.apply(x, bias, None, *weights)
        if tape._keep:
            # a private copy: the consumer may rework the output in place (the rotary embedding does, on q and k), and
            # the replay pass must hand back what the GEMM produced
            tape.store(y.detach().clone())
        return y
    return _LinearFn.apply(x, bias, tape.fetch(), *weights)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if _kernel_ok(x, weight) or (bias is None and not x.is_cuda and x.dtype == torch.bfloat16 and _cpu_fp8(x, [weight])):
        return _with_tape(x, bias, [weight], lambda: _LinearFn.apply(x, bias, None, weight))
    return _with_tape(x, bias, [weight], lambda: F.linear(x, weight, bias))


def linear_fused(x: torch.Tensor, weights: Sequence[torch.Tensor]) -> torch.Tensor:
    """``x @ cat(weights, 0).T`` as one ``[..., sum(N_i)]`` tensor."""
    if all(_kernel_ok(x, w) for w in weights):
        return _with_tape(x, None, weights, lambda: _LinearFn.apply(x, None, None, *weights))
    if not x.is_cuda and x.dtype == torch.bfloat16 and _cpu_fp8(x, weights):
        return torch.cat([_LinearFn.apply(x, None, None, w) for w in weights], dim=-1)
    return _with_tape(x, None, weights, lambda: torch.cat([F.linear(x, w) for w in weights], dim=-1))


# --------------------------------------------------------------------------------------------------------------
# gate | up projection with the SwiGLU activation in the GEMM epilogue
# --------------------------------------------------------------------------------------------------------------
from ctypes import c_int, c_longlong, c_void_p  # noqa: E402

_lib.register("fb_gemm2_swiglu", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                                  c_longlong, c_longlong, c_int, c_void_p])


class _GateUpSwiGLU(torch.autograd.Function):
    """``z = silu(x @ Wg.T) * (x @ Wu.T)`` from ONE kernel: the GEMM's epilogue holds gate_j and up_j of the same hidden
    index side by side (the two CTAs of a pair load the gate rows and the up rows of the fused weight), writes both (the
    backward pass needs them) and the activation.  Saves the pass that re-read ``[T, 2 I]`` to write ``[T, I]``."""

    @staticmethod
    def forward(ctx, x, wg, wu):
        from . import gemm as gemm_ops
        shape = x.shape
        K = shape[-1]
        x2 = x.reshape(-1, K)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        T, I = x2.shape[0], wg.shape[0]
        wcat = _cat_view([wg.detach(), wu.detach()])
        pend = gemm_ops.pending_gather()
        if pend is not None and not pend.done and pend.touches(wcat):
            pend.flush()
        gu = torch.empty(T, 2 * I, dtype=x.dtype, device=x.device)
        z = torch.empty(T, I, dtype=x.dtype, device=x.device)
        rc = _lib.lib().fb_gemm2_swiglu(x2.data_ptr(), wcat.data_ptr(), gu.data_ptr(), z.data_ptr(), T, I, K, x2.stride(0),
                                        wcat.stride(0), gu.stride(0), z.stride(0), gemm_ops._sm_count(x.device),
                                        _lib.stream_ptr())
        _lib.check(rc, "fb_gemm2_swiglu")
        _lib.count_launch()
        ctx.save_for_backward(x2, gu, wg, wu)
        ctx.params = (wg, wu)
        ctx.shape = shape
        return z.view(*shape[:-1], I)

    @staticmethod
    def backward(ctx, dz):
        from .activations import swiglu_backward
        x2, gu, wg, wu = ctx.saved_tensors
        I = wg.shape[0]
        dz2 = dz.reshape(-1, I)
        dgu = swiglu_backward(dz2 if dz2.is_contiguous() else dz2.contiguous(), gu)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dgu, _cat_view([wg, wu]) if _adjacent([wg, wu]) else torch.cat([wg, wu], 0)).view(ctx.shape)
        mgs = [getattr(w, "main_grad", None) for w in ctx.params]
        gg = gu_ = None
        if all(m is not None for m in mgs) and _adjacent(mgs):
            gemm_tn(dgu, x2, out=_cat_view(mgs), accumulate=True)
        elif all(m is not None for m in mgs):
            gemm_tn(dgu[:, :I], x2, out=mgs[0], accumulate=True)
            gemm_tn(dgu[:, I:], x2, out=mgs[1], accumulate=True)
        else:
            gg = gemm_tn(dgu[:, :I], x2, out_dtype=torch.float32).to(wg.dtype)
            gu_ = gemm_tn(dgu[:, I:], x2, out_dtype=torch.float32).to(wu.dtype)
        return dx, gg, gu_


def gate_up_swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor) -> Optional[torch.Tensor]:
    """The fused projection + activation when ``FLAME_B200_FUSED_SWIGLU=1`` and its conditions hold (bf16 on the GPU,
    adjacent weights, I a multiple of 128, no fp8 weights, no selective-checkpointing tape); ``None`` tells the caller to
    take the two-step path.  Opt-in because it measured slower: at 65,536 x 5632 x 1024 the GEMM with the activation in
    its epilogue takes 0.84 ms against 0.73 ms for the plain GEMM plus the SwiGLU kernel (the epilogue writes three
    tiles - gate, up and the product, which the backward needs - per accumulator instead of two, and that costs the
    pipeline more than the saved 0.7 GB read is worth)."""
    import os
    if not (_kernel_ok(x, wg) and _kernel_ok(x, wu) and wg.shape == wu.shape and wg.shape[0] % 128 == 0):
        return None
    if getattr(wg, "_fp8", False) or getattr(wu, "_fp8", False) or sac.current() is not None:
        return None
    if not _adjacent([wg.detach(), wu.detach()]) or os.environ.get("FLAME_B200_FUSED_SWIGLU", "0") != "1":
        return None
    return _GateUpSwiGLU.apply(x, wg, wu)
