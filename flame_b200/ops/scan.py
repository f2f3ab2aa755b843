"""State-space scans: Mamba selective scan and Mamba2 SSD (fla/layers/mamba.py:361-397, fla/layers/mamba2.py:585-669)."""
from __future__ import annotations

import torch

from . import linear_attn as la
from .varlen import VarlenMeta


def selective_scan(u, delta, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    return la.selective_scan(u, delta, A, B, C, D, meta)


def mamba2_ssd(x, dt, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    return la.mamba2_ssd(x, dt, A, B, C, D, meta)
