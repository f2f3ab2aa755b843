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
        # context parallelism cut the row inside documents: the transition of the delta rule is not diagonal, so the state
        # is not handed over; the rank recomputes the prefix of its first document from the owners' rows instead
        from ..parallel.context_parallel import borrow_prefix
        q, k, v, beta, g = borrow_prefix([q, k, v, beta, g], sl)
        return gated_delta_rule(q, k, v, beta, g, sl.ext_meta, scale, l2norm_qk)[sl.prefix:]
    if l2norm_qk:
        if _lib.available() and q.is_cuda and q.dtype == torch.bfloat16:
            from .chunk_kernels import l2norm
            q, k = l2norm(q), l2norm(k)
        else:
            q, k = la.l2norm(q), la.l2norm(k)
    return gated_delta_rule_tc(q, k, v, beta, g, meta, scale)
