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
    return gla_tc(q, k, v, g, meta, scale)


def gsa(q, k, v, s, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """Two chained passes (fla/ops/gsa/chunk.py:826-871): slots written with key k and value s under a value-side
    decay g; softmax over the slot read-out; values read through the slot memory with a key-side decay g."""
    from .chunked import gla_tc, gla_vdecay_tc
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    ok = gla_vdecay_tc(q, k, s, g, meta, scale)
    qv = torch.softmax(ok.float(), -1).to(v.dtype)
    return gla_tc(qv, s, v, g, meta, scale=1.0).to(v.dtype)
