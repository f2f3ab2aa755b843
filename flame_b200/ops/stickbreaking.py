"""Stick-breaking attention entry point: ``sb_attention(q, k, v, meta) -> (out, remainder)``.

Replaces ``sb_attn`` / ``sb_attn_varlen`` (custom_models/sba/stickbreaking_attention)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import linear_attn as la
from .varlen import VarlenMeta


def sb_attention(q, k, v, meta: VarlenMeta, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    return la.stickbreaking_reference(q, k, v, meta, scale)
