"""State-space scans: Mamba selective scan and Mamba2 SSD (fla/layers/mamba.py:361-397, fla/layers/mamba2.py:585-669)."""
from __future__ import annotations

import torch

from . import linear_attn as la
from .varlen import VarlenMeta


def selective_scan(u, delta, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    """Mamba-1 scan.  u, delta ``[T, Di]``; A ``[Di, N]``; B, C ``[T, N]``; D ``[Di]``:
    ``h_t = exp(delta_t A) h_{t-1} + delta_t B_t u_t``,  ``y_t = h_t C_t + D u_t``, the state reset at every document start.
    On CUDA with N = 16 the chunk-parallel kernels of ``csrc/sscan.cu`` run; otherwise the chunked torch formulation."""
    from . import _lib
    sl = getattr(meta, "sequence_slice", None)
    if sl is not None:   # context parallelism cut the row inside documents: recompute the first document's prefix
        from ..parallel.context_parallel import borrow_prefix
        u, delta, B, C = borrow_prefix([u, delta, B, C], sl)
        return selective_scan(u, delta, A, B, C, D, sl.ext_meta)[sl.prefix:]
    if _lib.available() and u.is_cuda and A.shape[1] == 16 and u.dtype == torch.bfloat16:
        from .chunk_kernels import SelectiveScan
        from .chunked import ChunkLayout
        lay = ChunkLayout.of(meta, 64)
        y = SelectiveScan.apply(lay.pack(u), lay.pack(delta.float()), A.float(), lay.pack(B.float()), lay.pack(C.float()),
                                D.float(), lay.first, lay.last)
        return lay.unpack(y)
    return la.selective_scan(u, delta, A, B, C, D, meta)


def mamba2_ssd(x, dt, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    """x [T, H, P], dt [T, H] (after softplus), A [H] (negative), B, C [T, G, N], D [H] -> y [T, H, P]:
    the SSD recurrence in its attention form (query C, key B, value dt * x, log decay A * dt) on ``chunked.scalar_gla_tc``."""
    from .gla import scalar_gla
    g = dt.float() * A.float()[None, :]
    xv = (x.float() * dt.float()[..., None]).to(x.dtype)
    y = scalar_gla(C.to(x.dtype), B.to(x.dtype), xv, g, meta, scale=1.0)   # B, C stay grouped: [T, G, N]
    return (y.float() + x.float() * D.float()[None, :, None]).to(x.dtype)
