"""Gated linear attention (per-channel key decay) and gated slot attention entry points.

``gla(q, k, v, g, meta)``: q, k ``[T, H, K]``, v ``[T, H, V]``, g ``[T, H, K]`` natural-log decays.
Replaces ``chunk_gla`` (fla/ops/gla/chunk.py:1080-1237) and ``chunk_gsa`` (fla/ops/gsa/chunk.py:826-943).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import linear_attn as la
from .varlen import VarlenMeta


def gla(q, k, v, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """Chunked GLA on the batched tcgen05 GEMM (``chunked.gla_tc``)."""
    from .chunked import gla_tc
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:
        return gla_state_passing(q, k, v, g, meta, scale, sl)
    return gla_tc(q, k, v, g, meta, scale)


def _vdecay_state_passing(q, k, v, gv, meta: VarlenMeta, scale: float, sl) -> torch.Tensor:
    """First pass of gated slot attention on a context-parallel slice: ``S_t = S_{t-1} diag(exp gv_t) + k_t v_t^T`` decays
    along the VALUE dimension, so the entering state contributes ``scale (q_t^T S_in) * exp(G_t)`` with ``G_t`` the cumulative
    log decay of the value channels, and a rank hands on ``A = exp(G_end)`` per value channel and
    ``B = sum_t k_t (v_t * exp(G_end - G_t))^T``.  Same protocol as ``gla_state_passing``."""
    from ..parallel.context_parallel import _AllGatherRows
    from .chunked import gla_vdecay_tc, ChunkLayout  # noqa: F401
    plain = VarlenMeta.from_cu_seqlens(meta.cu_cpu().to(torch.int32), int(meta.cu_cpu()[-1]), meta.device)
    o = gla_vdecay_tc(q, k, v, gv, plain, scale)                   # fp32 [T, H, dv], every local document from a zero state
    cu = meta.cu_cpu().tolist()
    gf = gv.float()
    a0 = cu[-2]
    G_last = gf[a0:].cumsum(0)                                     # [L, H, dv]
    A = G_last[-1].exp()                                           # [H, dv]
    vh = v[a0:].float() * (G_last[-1][None] - G_last).exp()
    B = torch.einsum("lhk,lhv->hkv", k[a0:].float(), vh)           # [H, dk, dv]
    A_all = _AllGatherRows.apply(A[None].contiguous(), sl.group)
    B_all = _AllGatherRows.apply(B[None].contiguous(), sl.group)
    s_in = None
    for j in range(sl.rank):
        leave = B_all[j]
        if sl.single[j] and s_in is not None:
            leave = leave + s_in * A_all[j][:, None, :]
        s_in = leave if sl.continues[j + 1] else None
    o = o + (A_all[:0].sum() + B_all[:0].sum()).to(o.dtype)        # empty slices: connected, independent of the values
    if s_in is not None:
        L1 = cu[1]
        G1 = gf[:L1].cumsum(0)
        corr = torch.einsum("lhk,hkv->lhv", q[:L1].float(), s_in) * G1.exp() * scale
        o = torch.cat([o[:L1] + corr.to(o.dtype), o[L1:]], 0)
    return o


def gla_state_passing(q, k, v, g, meta: VarlenMeta, scale: Optional[float], sl) -> torch.Tensor:
    """GLA on one rank's slice of a row that context parallelism cut inside documents (``sl``: the slice's
    ``SequenceSlice``; ``meta``: the slice's own document boundaries).

    ``S_t = diag(exp g_t) S_{t-1} + k_t v_t^T`` is linear in the state, so a rank can run its slice from a zero state and
    add what the state that enters its first document contributes: ``o_t += scale (q_t * exp(G_t))^T S_in`` with ``G_t`` the
    cumulative log decay from the slice's start.  What a rank hands on is the pair (decay ``A = exp(G_end)``, state ``B`` of
    its last document from a zero state); one all-gather of the pairs lets every rank chain its predecessors.  The
    gather is differentiable (its backward is a reduce-scatter), so the state's gradient reaches the ranks it came from.
    Counterpart of fla's state-passing context parallelism, which all-gathers an affine map per rank and folds the
    predecessors' maps into the initial state (fla/ops/cp/chunk_delta_h.py:42-318, host side :736-909)."""
    from ..parallel.context_parallel import _AllGatherRows
    from .chunked import gla_tc
    T, H, dk = q.shape
    scale = dk ** -0.5 if scale is None else scale
    o = gla_tc(q, k, v, g, meta, scale)                         # every local document from a zero state
    cu = meta.cu_cpu().tolist()
    gf = g.float()
    # the pair this rank hands on: its last document's local part
    a0 = cu[-2]
    G_last = gf[a0:].cumsum(0)                                   # [L, H, dk]
    A = G_last[-1].exp()                                         # [H, dk]
    khat = k[a0:].float() * (G_last[-1][None] - G_last).exp()
    B = torch.einsum("lhk,lhv->hkv", khat, v[a0:].float())       # [H, dk, dv]
    A_all = _AllGatherRows.apply(A[None].contiguous(), sl.group)  # [world, H, dk]
    B_all = _AllGatherRows.apply(B[None].contiguous(), sl.group)  # [world, H, dk, dv]
    # the state that enters each rank, chained from rank 0 up to this one
    s_in = None
    for j in range(sl.rank):
        leave = B_all[j]
        if sl.single[j] and s_in is not None:
            leave = leave + A_all[j][..., None] * s_in           # rank j's slice was the middle of one long document
        s_in = leave if sl.continues[j + 1] else None
    # every rank must take part in the gather's backward collective, also one that reads nobody's pair
    o = o + (A_all[:0].sum() + B_all[:0].sum()).to(o.dtype)   # empty slices: connected, independent of the values
    if s_in is not None:
        L1 = cu[1]
        G1 = gf[:L1].cumsum(0)
        corr = torch.einsum("lhk,hkv->lhv", q[:L1].float() * G1.exp(), s_in) * scale
        o = torch.cat([o[:L1] + corr.to(o.dtype), o[L1:]], 0)
    return o


def gsa(q, k, v, s, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """Two chained passes (fla/ops/gsa/chunk.py:826-871): slots written with key k and value s under a value-side
    decay g; softmax over the slot read-out; values read through the slot memory with a key-side decay g."""
    from .chunked import gla_tc, gla_vdecay_tc
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:
        # context parallelism cut the row inside documents: both passes are diagonal-decay recurrences, each hands its
        # state from rank to rank (the slot softmax between them is local to a token)
        K = q.shape[-1]
        scale = K ** -0.5 if scale is None else scale
        ok = _vdecay_state_passing(q, k, s, g, meta, scale, sl)
        qv = torch.softmax(ok.float(), -1).to(v.dtype)
        return gla_state_passing(qv, s, v, g, meta, 1.0, sl).to(v.dtype)
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    ok = gla_vdecay_tc(q, k, s, g, meta, scale)
    qv = torch.softmax(ok.float(), -1).to(v.dtype)
    return gla_tc(qv, s, v, g, meta, scale=1.0).to(v.dtype)


def scalar_gla(q, k, v, g, meta: VarlenMeta, scale: float = 1.0) -> torch.Tensor:
    """``S_t = exp(g_t) S_{t-1} + k_t v_t^T, o_t = scale q_t^T S_t`` with one log decay per head (Mamba2's SSD in its
    attention form): q, k ``[T, G, N]`` with G dividing H, v ``[T, H, P]``, g ``[T, H]``.  ``chunked.scalar_gla_tc``, with the
    state handed from rank to rank when context parallelism cut the row inside documents."""
    from .chunked import scalar_gla_tc
    sl = getattr(meta, "sequence_slice", None)
    if sl is None:
        return scalar_gla_tc(q, k, v, g, meta, scale)
    from ..parallel.context_parallel import _AllGatherRows
    T, G, N = q.shape
    H = v.shape[1]
    rep = H // G
    o = scalar_gla_tc(q, k, v, g, meta, scale)
    cu = meta.cu_cpu().tolist()
    gf = g.float()
    a0 = cu[-2]
    G_last = gf[a0:].cumsum(0)                                                     # [L, H]
    A = G_last[-1].exp()                                                           # [H]
    kh = k[a0:].float().repeat_interleave(rep, 1) * (G_last[-1][None] - G_last).exp()[..., None]
    B = torch.einsum("lhn,lhp->hnp", kh, v[a0:].float())                           # [H, N, P]
    A_all = _AllGatherRows.apply(A[None].contiguous(), sl.group)                   # [world, H]
    B_all = _AllGatherRows.apply(B[None].contiguous(), sl.group)                   # [world, H, N, P]
    s_in = None
    for j in range(sl.rank):
        leave = B_all[j]
        if sl.single[j] and s_in is not None:
            leave = leave + A_all[j][:, None, None] * s_in
        s_in = leave if sl.continues[j + 1] else None
    o = o + (A_all[:0].sum() + B_all[:0].sum()).to(o.dtype)   # empty slices: connected, independent of the values
    if s_in is not None:
        L1 = cu[1]
        G1 = gf[:L1].cumsum(0)
        qh = q[:L1].float().repeat_interleave(rep, 1) * G1.exp()[..., None]
        corr = torch.einsum("lhn,hnp->lhp", qh, s_in) * scale
        o = torch.cat([o[:L1] + corr.to(o.dtype), o[L1:]], 0)
    return o
