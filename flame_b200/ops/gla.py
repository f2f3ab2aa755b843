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
    return la.gla_chunk(q, k, v, g, meta, scale)


def gsa(q, k, v, s, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    return la.gsa_chunk(q, k, v, s, g, meta, scale)
