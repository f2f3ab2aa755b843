"""(Gated) delta rule entry point.

``gated_delta_rule(q, k, v, beta, g, meta)``: q, k ``[T, H, K]``, v ``[T, H, V]``, beta ``[T, H]``, g ``[T, H]`` natural-log
decay or None.  With ``l2norm_qk`` the L2 normalisation of q and k that the reference performs inside its kernel
is applied here.  Replaces ``chunk_delta_rule`` / ``chunk_gated_delta_rule``
(fla/ops/delta_rule/chunk.py:18-139, fla/ops/gated_delta_rule/chunk.py:29-235).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import linear_attn as la
from .varlen import VarlenMeta


def gated_delta_rule(q, k, v, beta, g, meta: VarlenMeta, scale: Optional[float] = None,
                     l2norm_qk: bool = True) -> torch.Tensor:
    from . import _lib
    from .chunked import gated_delta_rule_tc
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:
        import os
        how = os.environ.get("FLAME_B200_CP_DELTA", "auto")
        if how == "auto":
            # documents no longer than a slice: recomputing a borrowed prefix costs at most one document; longer ones:
            # only passing the state keeps a rank's work at its own slice
            how = "borrow" if 0 <= sl.max_prefix <= sl.hi - sl.lo else "state"
        if how == "borrow":
            # the other exact way: recompute the prefix of the slice's first document from the owners' rows
            from ..parallel.context_parallel import borrow_prefix
            q, k, v, beta, g = borrow_prefix([q, k, v, beta, g], sl)
            return gated_delta_rule(q, k, v, beta, g, sl.ext_meta, scale, l2norm_qk)[sl.prefix:]
        return _delta_rule_state_passing(q, k, v, beta, g, meta, scale, l2norm_qk, sl)
    if l2norm_qk:
        if _lib.available() and q.is_cuda and q.dtype == torch.bfloat16:
            from .chunk_kernels import l2norm
            q, k = l2norm(q), l2norm(k)
        else:
            q, k = la.l2norm(q), la.l2norm(k)
    return gated_delta_rule_tc(q, k, v, beta, g, meta, scale)


def _delta_rule_state_passing(q, k, v, beta, g, meta: VarlenMeta, scale, l2norm_qk: bool, sl) -> torch.Tensor:
    """The (gated) delta rule on one rank's slice of a row that context parallelism cut inside documents.

    The state update ``S' = alpha S - beta k (k^T S) + beta k v^T`` is affine in the state, with a transition that is not
    diagonal, so a rank hands on an affine map: the state ``B`` its last document leaves from a zero state and the
    transition ``P`` (``dk x dk``), ``S_end = P S_in + B`` (the ``[K, V + K]`` map of fla/ops/cp/chunk_delta_h.py:42-318).
    Both are obtained from the ORDINARY operator, because the delta rule is an associative memory: a token with key
    ``e_i``, ``beta = 1`` and value ``x`` sets row ``i`` of the state to ``x``, and a token with query ``e_i`` and
    ``beta = 0`` reads row ``i`` back.

    * pair of the last document: ``dk`` writing tokens that set the right ``dk`` columns of a state widened to
      ``dv + dk`` columns to the identity, then the document's local tokens with values ``[v | 0]``, then ``dk`` reading
      tokens: what they read is ``[B | P]``;
    * after one differentiable all-gather of the pairs every rank chains its predecessors
      (``S_in[j+1] = P_j S_in[j] + B_j`` while the document goes on) and runs its slice with ``dk`` writing tokens in
      front of its first document whose values are the rows of ``S_in``.

    Every rank works on its own slice plus ``3 dk`` tokens and one more pass over its last document, whatever the length
    of the documents (a single document across all ranks included)."""
    from ..parallel.context_parallel import _AllGatherRows
    T, H, dk = q.shape
    dv = v.shape[-1]
    dev, dt = q.device, q.dtype
    scale = dk ** -0.5 if scale is None else scale
    cu = meta.cu_cpu().tolist()
    eye = torch.eye(dk, device=dev, dtype=dt)[:, None, :].expand(dk, H, dk)          # token i carries e_i for every head
    zeros_k = torch.zeros(dk, H, dk, device=dev, dtype=dt)
    ones_b = torch.ones(dk, H, device=dev, dtype=beta.dtype)
    zeros_b = torch.zeros(dk, H, device=dev, dtype=beta.dtype)
    zeros_g = None if g is None else torch.zeros(dk, H, device=dev, dtype=g.dtype)

    def one_doc(n: int) -> VarlenMeta:
        return VarlenMeta.from_cu_seqlens(torch.tensor([0, n], dtype=torch.int32), n, dev)

    # ---- the pair (B, P) of the last document's local part ------------------------------------------------------
    a0 = cu[-2]
    L = T - a0
    wide = lambda left, right: torch.cat([left, right], -1)                           # noqa: E731
    q_seq = torch.cat([zeros_k, torch.zeros(L, H, dk, device=dev, dtype=dt), eye], 0)
    k_seq = torch.cat([eye, k[a0:], eye], 0)
    v_seq = torch.cat([wide(torch.zeros(dk, H, dv, device=dev, dtype=dt), eye),
                       wide(v[a0:], torch.zeros(L, H, dk, device=dev, dtype=dt)),
                       torch.zeros(dk, H, dv + dk, device=dev, dtype=dt)], 0)
    beta_seq = torch.cat([ones_b, beta[a0:], zeros_b], 0)
    g_seq = None if g is None else torch.cat([zeros_g, g[a0:], zeros_g], 0)
    read = gated_delta_rule(q_seq, k_seq, v_seq, beta_seq, g_seq, one_doc(L + 2 * dk), 1.0, l2norm_qk)[-dk:]
    S_end = read.float().permute(1, 0, 2)                                             # [H, dk, dv + dk]
    B, P = S_end[..., :dv], S_end[..., dv:]
    B_all = _AllGatherRows.apply(B[None].contiguous(), sl.group)                      # [world, H, dk, dv]
    P_all = _AllGatherRows.apply(P[None].contiguous(), sl.group)                      # [world, H, dk, dk]
    s_in = None
    for j in range(sl.rank):
        leave = B_all[j]
        if sl.single[j] and s_in is not None:
            leave = leave + P_all[j] @ s_in                                           # rank j lies inside one long document
        s_in = leave if sl.continues[j + 1] else None
    connect = (B_all[:0].sum() + P_all[:0].sum()).to(dt)   # empty slices: every rank joins the gathers' backward collective
    # ---- the slice itself, its first document started from S_in ---------------------------------------------------
    if s_in is None:
        return gated_delta_rule(q, k, v, beta, g, _plain(meta), scale, l2norm_qk) + connect
    rows = s_in.permute(1, 0, 2).to(dt)                                               # [dk, H, dv]: token i writes row i
    q_m = torch.cat([zeros_k, q], 0)
    k_m = torch.cat([eye, k], 0)
    v_m = torch.cat([rows, v], 0)
    beta_m = torch.cat([ones_b, beta], 0)
    g_m = None if g is None else torch.cat([zeros_g, g], 0)
    cu_m = torch.tensor([0] + [c + dk for c in cu[1:]], dtype=torch.int32)
    meta_m = VarlenMeta.from_cu_seqlens(cu_m, T + dk, dev)
    return gated_delta_rule(q_m, k_m, v_m, beta_m, g_m, meta_m, scale, l2norm_qk)[dk:] + connect


def _plain(meta: VarlenMeta) -> VarlenMeta:
    """The slice's own document boundaries without the context-parallel annotations."""
    return VarlenMeta.from_cu_seqlens(meta.cu_cpu().to(torch.int32), int(meta.cu_cpu()[-1]), meta.device)
