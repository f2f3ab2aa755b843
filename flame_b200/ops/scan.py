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
    if sl is not None:
        return _selective_scan_state_passing(u, delta, A, B, C, D, meta, sl)
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


def _selective_scan_state_passing(u, delta, A, B, C, D, meta: VarlenMeta, sl) -> torch.Tensor:
    """Mamba-1's scan on one rank's slice of a row that context parallelism cut inside documents.  The state
    ``h_t[d, n] = exp(delta_t[d] A[d, n]) h_{t-1}[d, n] + delta_t[d] B_t[n] u_t[d]`` decays per element, so a rank hands on
    the pair (``exp(A * sum delta)``, state of its last document from a zero state) and adds
    ``sum_n C_t[n] exp(A[d, n] cumsum(delta)_t[d]) h_in[d, n]`` to the rows of its first document; the pairs travel in one
    differentiable all-gather (same protocol as ``gla.gla_state_passing``).  The ``[tokens, Di]`` terms are formed one
    state index at a time, so nothing of size ``tokens x Di x N`` is materialised."""
    from ..parallel.context_parallel import _AllGatherRows
    N = A.shape[1]
    plain = VarlenMeta.from_cu_seqlens(meta.cu_cpu().to(torch.int32), int(meta.cu_cpu()[-1]), meta.device)
    y = selective_scan(u, delta, A, B, C, D, plain)                      # every local document from a zero state
    cu = meta.cu_cpu().tolist()
    Af, df = A.float(), delta.float()
    a0 = cu[-2]
    c_last = df[a0:].cumsum(0)                                            # [L, Di]
    total = c_last[-1]                                                    # [Di]
    dec = (Af * total[:, None]).exp()                                     # [Di, N]
    du = df[a0:] * u[a0:].float()                                         # [L, Di]
    Bf = B[a0:].float()
    h_end = torch.stack([((Af[:, n][None] * (total[None] - c_last)).exp() * du * Bf[:, n:n + 1]).sum(0) for n in range(N)], -1)
    dec_all = _AllGatherRows.apply(dec[None].contiguous(), sl.group)      # [world, Di, N]
    h_all = _AllGatherRows.apply(h_end[None].contiguous(), sl.group)      # [world, Di, N]
    h_in = None
    for j in range(sl.rank):
        leave = h_all[j]
        if sl.single[j] and h_in is not None:
            leave = leave + dec_all[j] * h_in
        h_in = leave if sl.continues[j + 1] else None
    y = y + (dec_all[:0].sum() + h_all[:0].sum()).to(y.dtype)             # empty slices: connected, independent of the values
    if h_in is not None:
        L1 = cu[1]
        c1 = df[:L1].cumsum(0)                                            # [L1, Di]
        Cf = C[:L1].float()
        corr = sum((Af[:, n][None] * c1).exp() * h_in[:, n][None] * Cf[:, n:n + 1] for n in range(N))
        y = torch.cat([y[:L1] + corr.to(y.dtype), y[L1:]], 0)
    return y
