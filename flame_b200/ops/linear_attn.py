"""Linear-attention / state-space token mixers on packed sequences: PyTorch formulations.

Every function takes packed tensors (``[T, H, ...]``) plus the batch's ``VarlenMeta`` and never lets state cross
a document boundary.  Two kinds of implementation live here:

* ``*_recurrent``: the token-by-token definition (fp32).  These are the test oracles; they restate the math of
  fla/ops/gla/naive.py:15-44, fla/ops/gated_delta_rule/naive.py:13-66, fla/ops/delta_rule/naive.py:12-37,
  fla/ops/gsa/naive.py:12-72, fla/layers/mamba.py:361-397 and fla/layers/mamba2.py:585-669.
* ``*_chunk``: chunk-parallel forms (chunk = 64 tokens, fp32 state, batched matmuls over all documents at
  once) that are differentiable through autograd.  They are the execution path wherever no hand-written
  kernel exists yet, and the CPU path of the plumbing configuration.

Gates are natural-log decays (``g <= 0``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .varlen import VarlenMeta

CHUNK = 64


# ----------------------------------------------------------------------------------------------------
# packing helpers: [T, ...] <-> [N, Lp, ...] with Lp a multiple of the chunk size
# ----------------------------------------------------------------------------------------------------
def _pad_plan(meta: VarlenMeta, chunk: int = CHUNK):
    key = ("pad_plan", chunk)
    plan = meta.cache.get(key)
    if plan is None:
        lens = meta.lengths_list()
        n = len(lens)
        lp = max(1, (max(lens) + chunk - 1) // chunk) * chunk if lens else chunk
        dev = meta.device
        cu = meta.cu_seqlens.long()
        ar = torch.arange(lp, device=dev)
        lens_t = (cu[1:] - cu[:-1])
        valid = ar[None, :] < lens_t[:, None]  # [N, Lp]
        src = (cu[:-1, None] + ar[None, :]).clamp_max(max(meta.total_tokens - 1, 0))
        plan = (n, lp, valid, src, valid.reshape(-1).nonzero().flatten())
        meta.cache[key] = plan
    return plan


def pack_to_padded(x: torch.Tensor, meta: VarlenMeta, chunk: int = CHUNK) -> torch.Tensor:
    """[T, ...] -> [N, Lp, ...] (zero padded)."""
    n, lp, valid, src, _ = _pad_plan(meta, chunk)
    out = x[src.reshape(-1)].reshape(n, lp, *x.shape[1:])
    mask = valid.reshape(n, lp, *([1] * (x.dim() - 1)))
    return out * mask.to(out.dtype)


def padded_to_pack(y: torch.Tensor, meta: VarlenMeta, chunk: int = CHUNK) -> torch.Tensor:
    """[N, Lp, ...] -> [T, ...]."""
    n, lp, valid, src, flat_idx = _pad_plan(meta, chunk)
    return y.reshape(n * lp, *y.shape[2:])[flat_idx]


def _doc_slices(meta: VarlenMeta):
    cu = meta.cu_cpu().tolist()
    return [(a, b) for a, b in zip(cu[:-1], cu[1:]) if b > a]


# ----------------------------------------------------------------------------------------------------
# GLA (per-channel decay on the key dimension); HGRN2 and GSA reuse it
# ----------------------------------------------------------------------------------------------------
def gla_recurrent(q, k, v, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """o_t = (scale q_t)^T S_t,  S_t = diag(exp g_t) S_{t-1} + k_t v_t^T  (per head, reset per document)."""
    T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qf, kf, vf, gf = (t.float() for t in (q, k, v, g))
    o = torch.zeros(T, H, V, dtype=torch.float32, device=q.device)
    for a, b in _doc_slices(meta):
        S = torch.zeros(H, K, V, dtype=torch.float32, device=q.device)
        for t in range(a, b):
            S = S * gf[t].exp()[..., None] + kf[t][..., None] * vf[t][:, None, :]
            o[t] = torch.einsum("hk,hkv->hv", qf[t] * scale, S)
    return o.to(v.dtype)


def gla_chunk(q, k, v, g, meta: VarlenMeta, scale: Optional[float] = None, chunk: int = CHUNK) -> torch.Tensor:
    """Chunk-parallel GLA.  Intra-chunk scores use 16-row sub-blocks re-based on the sub-block's first row so
    that no exponent is ever positive (the "secondary chunking" of fla/ops/gla/chunk.py:88-170)."""
    T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    out_dtype = v.dtype
    qp, kp, vp, gp = (pack_to_padded(t.float(), meta, chunk) for t in (q, k, v, g))
    N, Lp = qp.shape[:2]
    NC = Lp // chunk
    # [N, NC, C, H, *] -> [N, H, NC, C, *]
    shp = lambda t: t.reshape(N, NC, chunk, H, -1).permute(0, 3, 1, 2, 4)
    qc, kc, vc, gc = shp(qp), shp(kp), shp(vp), shp(gp)
    b = gc.cumsum(3)  # within-chunk cumulative log decay (<= 0, decreasing)
    b_last = b[:, :, :, -1:, :]
    # ---- inter-chunk state recurrence (sequential over chunks, batched over documents and heads)
    k_dec = kc * (b_last - b).exp()  # key contribution decayed to the end of its chunk
    S = torch.zeros(N, H, K, V, dtype=torch.float32, device=q.device)
    states = []
    for c in range(NC):
        states.append(S)
        S = S * b_last[:, :, c, 0, :, None].exp() + torch.einsum("nhck,nhcv->nhkv", k_dec[:, :, c], vc[:, :, c])
    S_all = torch.stack(states, 2)  # [N, H, NC, K, V] state at chunk start
    o_inter = torch.einsum("nhcik,nhckv->nhciv", qc * b.exp(), S_all)
    # ---- intra-chunk: A_ij = sum_d q_id k_jd exp(b_id - b_jd), j <= i
    BC = 16
    NB = chunk // BC
    A = torch.zeros(N, H, NC, chunk, chunk, dtype=torch.float32, device=q.device)
    for i in range(NB):
        rows = slice(i * BC, (i + 1) * BC)
        b_n = b[:, :, :, i * BC: i * BC + 1, :]  # first row of the query sub-block
        q_i = qc[:, :, :, rows] * (b[:, :, :, rows] - b_n).exp()
        if i > 0:
            cols = slice(0, i * BC)
            k_j = kc[:, :, :, cols] * (b_n - b[:, :, :, cols]).exp()
            A[:, :, :, rows, cols] = torch.einsum("nhcik,nhcjk->nhcij", q_i, k_j)
        # diagonal sub-block: pairwise exponent differences, masked to j <= i
        d = b[:, :, :, rows, None, :] - b[:, :, :, None, rows, :]  # [.., BC, BC, K]
        tri = torch.tril(torch.ones(BC, BC, dtype=torch.bool, device=q.device))
        d = d.masked_fill(~tri[..., None], float("-inf"))
        A[:, :, :, rows, rows] = torch.einsum("nhcik,nhcjk,nhcijk->nhcij", qc[:, :, :, rows], kc[:, :, :, rows], d.exp())
    o_intra = torch.einsum("nhcij,nhcjv->nhciv", A, vc)
    o = (o_inter + o_intra) * scale
    o = o.permute(0, 2, 3, 1, 4).reshape(N, Lp, H, V)
    return padded_to_pack(o, meta, chunk).to(out_dtype)


# ----------------------------------------------------------------------------------------------------
# scalar-gated linear attention (one decay per head and step): Mamba2 SSD and the gated delta rule share it
# ----------------------------------------------------------------------------------------------------
def _chunk_views(meta, chunk, H, *ts):
    out = []
    for t in ts:
        p = pack_to_padded(t.float(), meta, chunk)
        N, Lp = p.shape[:2]
        NC = Lp // chunk
        out.append(p.reshape(N, NC, chunk, H, -1).permute(0, 3, 1, 2, 4))
    return out


def scalar_gla_chunk(q, k, v, g, meta: VarlenMeta, scale: float = 1.0, chunk: int = CHUNK) -> torch.Tensor:
    """o_t = scale q_t^T S_t,  S_t = exp(g_t) S_{t-1} + k_t v_t^T with g [T, H]."""
    T, H, K = q.shape
    V = v.shape[-1]
    qc, kc, vc, gc = _chunk_views(meta, chunk, H, q, k, v, g[..., None])
    N, _, NC = qc.shape[:3]
    b = gc.cumsum(3)  # [N, H, NC, C, 1]
    b_last = b[:, :, :, -1:, :]
    k_dec = kc * (b_last - b).exp()
    S = torch.zeros(N, H, K, V, dtype=torch.float32, device=q.device)
    states = []
    for c in range(NC):
        states.append(S)
        S = S * b_last[:, :, c, 0, :, None].exp() + torch.einsum("nhck,nhcv->nhkv", k_dec[:, :, c], vc[:, :, c])
    S_all = torch.stack(states, 2)
    o_inter = torch.einsum("nhcik,nhckv->nhciv", qc * b.exp(), S_all)
    diff = b - b.transpose(3, 4)  # [N,H,NC,C,C]: b_i - b_j
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    decay = diff.masked_fill(~tri, float("-inf")).exp()
    A = torch.einsum("nhcik,nhcjk->nhcij", qc, kc) * decay
    o = (o_inter + torch.einsum("nhcij,nhcjv->nhciv", A, vc)) * scale
    Lp = NC * chunk
    o = o.permute(0, 2, 3, 1, 4).reshape(N, Lp, H, V)
    return padded_to_pack(o, meta, chunk).to(v.dtype)


# ----------------------------------------------------------------------------------------------------
# (gated) delta rule
# ----------------------------------------------------------------------------------------------------
def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def gated_delta_rule_recurrent(q, k, v, beta, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """S <- S exp(g_t);  v' = (v_t - S^T k_t) beta_t;  S <- S + k_t v'^T;  o_t = S^T (scale q_t).
    g may be None (plain delta rule).  q and k are expected already normalised."""
    T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    gf = g.float() if g is not None else None
    o = torch.zeros(T, H, V, dtype=torch.float32, device=q.device)
    for a, b in _doc_slices(meta):
        S = torch.zeros(H, K, V, dtype=torch.float32, device=q.device)
        for t in range(a, b):
            if gf is not None:
                S = S * gf[t].exp()[:, None, None]
            vn = (vf[t] - torch.einsum("hkv,hk->hv", S, kf[t])) * bf[t][:, None]
            S = S + kf[t][..., None] * vn[:, None, :]
            o[t] = torch.einsum("hkv,hk->hv", S, qf[t] * scale)
    return o.to(v.dtype)


def gated_delta_rule_chunk(q, k, v, beta, g, meta: VarlenMeta, scale: Optional[float] = None,
                           chunk: int = CHUNK) -> torch.Tensor:
    """Chunk-parallel (gated) delta rule through the WY representation:
    A = strict_tril(beta_i (k_i . k_j) exp(b_i - b_j)),  T = (I + A)^-1,  u = T (beta v),  w = T (beta exp(b) k);
    per chunk  v_new = u - w S,  S' = exp(b_last) S + k^T (v_new exp(b_last - b)),
    o = scale [ (q S) exp(b) + tril((q k^T) exp(b_i - b_j)) v_new ]."""
    T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    if g is None:
        g = torch.zeros(T, H, dtype=torch.float32, device=q.device)
    qc, kc, vc, bc, gc = _chunk_views(meta, chunk, H, q, k, v, beta[..., None], g[..., None])
    N, _, NC = qc.shape[:3]
    b = gc.cumsum(3)  # [N,H,NC,C,1]
    b_last = b[:, :, :, -1:, :]
    diff = b - b.transpose(3, 4)
    eye = torch.eye(chunk, dtype=torch.float32, device=q.device)
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    kk = torch.einsum("nhcik,nhcjk->nhcij", kc, kc)
    A = (bc * kk * diff.masked_fill(~strict, float("-inf")).exp())
    # (I + A) X = rhs with unit lower-triangular I + A
    rhs = torch.cat([bc * vc, bc * b.exp() * kc], dim=-1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
    u, w = sol[..., :V], sol[..., V:]
    qk = torch.einsum("nhcik,nhcjk->nhcij", qc, kc) * diff.masked_fill(~tri, float("-inf")).exp()
    S = torch.zeros(N, H, K, V, dtype=torch.float32, device=q.device)
    outs = []
    for c in range(NC):
        v_new = u[:, :, c] - torch.einsum("nhik,nhkv->nhiv", w[:, :, c], S)
        o_c = torch.einsum("nhik,nhkv->nhiv", qc[:, :, c] * b[:, :, c].exp(), S) + torch.einsum(
            "nhij,nhjv->nhiv", qk[:, :, c], v_new)
        outs.append(o_c)
        S = S * b_last[:, :, c, 0, :, None].exp() + torch.einsum(
            "nhik,nhiv->nhkv", kc[:, :, c], v_new * (b_last[:, :, c] - b[:, :, c]).exp())
    o = torch.stack(outs, 2) * scale
    Lp = NC * chunk
    o = o.permute(0, 2, 3, 1, 4).reshape(N, Lp, H, V)
    return padded_to_pack(o, meta, chunk).to(v.dtype)


def gdn_gate(a: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    """g = -exp(A_log) * softplus(a + dt_bias)   (fla/ops/gated_delta_rule/gate.py:20-44)."""
    return -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())


# ----------------------------------------------------------------------------------------------------
# GSA: keys -> slots -> softmax over slots -> values
# ----------------------------------------------------------------------------------------------------
def gsa_recurrent(q, k, v, s, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    T, H, K = q.shape
    scale = K ** -0.5 if scale is None else scale
    ok = gla_recurrent_vdecay(q, k, s, g, meta, scale)
    qv = torch.softmax(ok.float(), -1)
    return gla_recurrent(qv, s, v, g, meta, scale=1.0).to(v.dtype)


def gla_recurrent_vdecay(q, k, v, gv, meta: VarlenMeta, scale: float) -> torch.Tensor:
    """State decays along its VALUE dimension: S_t = S_{t-1} diag(exp gv_t) + k_t v_t^T."""
    T, H, K = q.shape
    V = v.shape[-1]
    qf, kf, vf, gf = (t.float() for t in (q, k, v, gv))
    o = torch.zeros(T, H, V, dtype=torch.float32, device=q.device)
    for a, b in _doc_slices(meta):
        S = torch.zeros(H, K, V, dtype=torch.float32, device=q.device)
        for t in range(a, b):
            S = S * gf[t].exp()[:, None, :] + kf[t][..., None] * vf[t][:, None, :]
            o[t] = torch.einsum("hk,hkv->hv", qf[t] * scale, S)
    return o


def gla_chunk_vdecay(q, k, v, gv, meta: VarlenMeta, scale: float, chunk: int = CHUNK) -> torch.Tensor:
    """Chunked form of ``gla_recurrent_vdecay``: the value-side decay factors out of the sum over keys, so
    o_t = exp(b_t) * sum_{s<=t} (q_t.k_s) v_s exp(-b_s) is evaluated per sub-block with re-basing."""
    T, H, K = q.shape
    V = v.shape[-1]
    qc, kc, vc, gc = _chunk_views(meta, chunk, H, q, k, v, gv)
    N, _, NC = qc.shape[:3]
    b = gc.cumsum(3)  # [N,H,NC,C,V]
    b_last = b[:, :, :, -1:, :]
    v_dec = vc * (b_last - b).exp()
    S = torch.zeros(N, H, K, V, dtype=torch.float32, device=q.device)
    states = []
    for c in range(NC):
        states.append(S)
        S = S * b_last[:, :, c, 0, None, :].exp() + torch.einsum("nhck,nhcv->nhkv", kc[:, :, c], v_dec[:, :, c])
    S_all = torch.stack(states, 2)
    o_inter = torch.einsum("nhcik,nhckv->nhciv", qc, S_all) * b.exp()
    qk = torch.einsum("nhcik,nhcjk->nhcij", qc, kc)
    BC = 16
    NB = chunk // BC
    o_intra = torch.zeros_like(o_inter)
    tri = torch.tril(torch.ones(BC, BC, dtype=torch.bool, device=q.device))
    for i in range(NB):
        rows = slice(i * BC, (i + 1) * BC)
        b_n = b[:, :, :, i * BC: i * BC + 1, :]
        acc = torch.zeros_like(o_inter[:, :, :, rows])
        if i > 0:
            cols = slice(0, i * BC)
            v_j = vc[:, :, :, cols] * (b_n - b[:, :, :, cols]).exp()
            acc = torch.einsum("nhcij,nhcjv->nhciv", qk[:, :, :, rows, cols], v_j) * (b[:, :, :, rows] - b_n).exp()
        d = (b[:, :, :, rows, None, :] - b[:, :, :, None, rows, :]).masked_fill(~tri[..., None], float("-inf")).exp()
        acc = acc + torch.einsum("nhcij,nhcjv,nhcijv->nhciv", qk[:, :, :, rows, rows], vc[:, :, :, rows], d)
        o_intra[:, :, :, rows] = acc
    o = (o_inter + o_intra) * scale
    Lp = NC * chunk
    o = o.permute(0, 2, 3, 1, 4).reshape(N, Lp, H, V)
    return padded_to_pack(o, meta, chunk)


def gsa_chunk(q, k, v, s, g, meta: VarlenMeta, scale: Optional[float] = None) -> torch.Tensor:
    """Two chained passes (fla/ops/gsa/chunk.py:826-871): slots written with key k and value s under a value-side
    decay g; softmax over the slot read-out; values read through the slot memory with a key-side decay g."""
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    ok = gla_chunk_vdecay(q, k, s, g, meta, scale)
    qv = torch.softmax(ok.float(), -1)
    return gla_chunk(qv, s, v, g, meta, scale=1.0).to(v.dtype)


# ----------------------------------------------------------------------------------------------------
# short causal depthwise convolution on packed sequences
# ----------------------------------------------------------------------------------------------------
def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], meta: VarlenMeta,
               activation: Optional[str] = "silu") -> torch.Tensor:
    """x [T, D]; weight [D, 1, W] (nn.Conv1d depthwise layout); taps never cross a document boundary
    (fla/modules/conv/triton/kernels.py:66-74)."""
    T, D = x.shape
    W = weight.shape[-1]
    pos = meta.position_ids.long()
    xf = x.float()
    wf = weight.float().reshape(D, W)
    y = xf * wf[:, W - 1]
    for j in range(1, W):
        shifted = torch.zeros_like(xf)
        shifted[j:] = xf[:-j]
        ok = (pos >= j).to(xf.dtype)[:, None]
        y = y + shifted * ok * wf[:, W - 1 - j]
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype)


# ----------------------------------------------------------------------------------------------------
# Mamba2 SSD and Mamba selective scan
# ----------------------------------------------------------------------------------------------------
def mamba2_ssd(x, dt, A, B, C, D, meta: VarlenMeta, chunk: int = CHUNK) -> torch.Tensor:
    """x [T, H, P], dt [T, H] (after softplus), A [H] (negative), B, C [T, G, N], D [H] -> y [T, H, P].
    h_t = exp(A dt_t) h_{t-1} + dt_t B_t x_t^T;  y_t = C_t h_t + D x_t  (fla/layers/mamba2.py:585-669)."""
    T, H, P = x.shape
    G = B.shape[1]
    rep = H // G
    Bh = B.repeat_interleave(rep, 1)
    Ch = C.repeat_interleave(rep, 1)
    g = dt.float() * A.float()[None, :]
    y = scalar_gla_chunk(Ch, Bh, x.float() * dt.float()[..., None], g, meta, scale=1.0, chunk=chunk)
    return (y.float() + x.float() * D.float()[None, :, None]).to(x.dtype)


def mamba2_ssd_recurrent(x, dt, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    Bh = B.repeat_interleave(rep, 1).float()
    Ch = C.repeat_interleave(rep, 1).float()
    xf, dtf = x.float(), dt.float()
    y = torch.zeros(T, H, P, dtype=torch.float32, device=x.device)
    for a, b in _doc_slices(meta):
        h = torch.zeros(H, N, P, dtype=torch.float32, device=x.device)
        for t in range(a, b):
            h = h * (A.float() * dtf[t]).exp()[:, None, None] + (dtf[t][:, None] * Bh[t])[..., None] * xf[t][:, None, :]
            y[t] = torch.einsum("hn,hnp->hp", Ch[t], h)
    return (y + xf * D.float()[None, :, None]).to(x.dtype)


def selective_scan(u, delta, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    """Mamba-1 scan.  u, delta [T, Di]; A [Di, N]; B, C [T, N]; D [Di].
    h_t = exp(delta_t A) h_{t-1} + delta_t B_t u_t;  y_t = h_t C_t + D u_t  (fla/layers/mamba.py:361-397).
    Evaluated in 64-step chunks: inside a chunk the decays are re-based on the chunk's first step, so every
    exponent is <= 0."""
    T, Di = u.shape
    N = A.shape[1]
    chunk = 64
    uf, df, Af, Bf, Cf = u.float(), delta.float(), A.float(), B.float(), C.float()
    up, dp, Bp, Cp = (pack_to_padded(t, meta, chunk) for t in (uf, df, Bf, Cf))
    Nd, Lp = up.shape[:2]
    NC = Lp // chunk
    h = torch.zeros(Nd, Di, N, dtype=torch.float32, device=u.device)
    ys = []
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=u.device))
    for c in range(NC):
        sl = slice(c * chunk, (c + 1) * chunk)
        dc, uc, Bc, Cc = dp[:, sl], up[:, sl], Bp[:, sl], Cp[:, sl]
        cum = dc.cumsum(1)  # [Nd, C, Di]
        # contribution of the carried state: y_t += C_t . (exp(A cum_t) h)
        dec = (cum[..., None] * Af).exp()  # [Nd, C, Di, N]
        y_c = torch.einsum("ncdk,ndk,nck->ncd", dec, h, Cc)
        # intra-chunk: sum_{s<=t} exp(A (cum_t - cum_s)) delta_s B_s u_s . C_t, pairwise so exponents stay <= 0
        diff = cum[:, :, None, :] - cum[:, None, :, :]  # [Nd, t, s, Di]
        diff = diff.masked_fill(~tri[None, :, :, None], 0.0)
        keep = tri[None, :, :, None].to(diff.dtype)
        # memory-light evaluation: loop over state dims
        acc = torch.zeros_like(y_c)
        du = dc * uc  # [Nd, C, Di]
        for kdim in range(N):
            e = (diff * Af[:, kdim]).exp() * keep  # [Nd, t, s, Di]
            acc = acc + torch.einsum("ntsd,nsd,ns,nt->ntd", e, du, Bc[..., kdim], Cc[..., kdim])
        y_c = y_c + acc
        ys.append(y_c)
        # carry the state to the end of the chunk
        last = cum[:, -1:, :]
        h = h * (last[:, 0, :, None] * Af).exp() + torch.einsum(
            "nsdk,nsd,nsk->ndk", ((last - cum)[..., None] * Af).exp(), du, Bc)
    y = torch.cat(ys, 1)
    y = padded_to_pack(y, meta, chunk) + uf * D.float()
    return y.to(u.dtype)


def selective_scan_recurrent(u, delta, A, B, C, D, meta: VarlenMeta) -> torch.Tensor:
    T, Di = u.shape
    N = A.shape[1]
    uf, df, Af, Bf, Cf = u.float(), delta.float(), A.float(), B.float(), C.float()
    y = torch.zeros(T, Di, dtype=torch.float32, device=u.device)
    for a, b in _doc_slices(meta):
        h = torch.zeros(Di, N, dtype=torch.float32, device=u.device)
        for t in range(a, b):
            h = h * (df[t][:, None] * Af).exp() + (df[t] * uf[t])[:, None] * Bf[t][None, :]
            y[t] = h @ Cf[t]
    return (y + uf * D.float()).to(u.dtype)


# ----------------------------------------------------------------------------------------------------
# stick-breaking attention
# ----------------------------------------------------------------------------------------------------
def stickbreaking_reference(q, k, v, meta: VarlenMeta, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """att_ij = sigmoid(l_ij) * prod_{j<m<i} (1 - sigmoid(l_im)) for j < i (strictly causal);
    returns (att @ v, 1 - sum_j att_ij)   (custom_models/sba/stickbreaking_attention/sb_ref.py:8-25)."""
    T, H, Dh = q.shape
    scale = 1.0 / math.sqrt(Dh) if scale is None else scale
    out = torch.zeros(T, H, Dh, dtype=torch.float32, device=q.device)
    rem = torch.ones(T, H, dtype=torch.float32, device=q.device)
    for a, b in _doc_slices(meta):
        L = b - a
        qq, kk, vv = (t[a:b].transpose(0, 1).float() for t in (q, k, v))
        logits = torch.matmul(qq, kk.transpose(1, 2)) * scale
        idx = torch.arange(L, device=q.device)
        mask = idx[None, :] >= idx[:, None]  # j >= i is masked
        log_z = F.logsigmoid(logits).masked_fill(mask, float("-inf"))
        log_beta = F.logsigmoid(-logits).masked_fill(mask, 0.0)
        # sum over m in (j, i): reverse cumulative sum along j, excluding j itself
        rc = log_beta.flip(-1).cumsum(-1).flip(-1) - log_beta
        att = (log_z + rc).exp()
        out[a:b] = torch.matmul(att, vv).transpose(0, 1)
        rem[a:b] = (1 - att.sum(-1)).transpose(0, 1)
    return out.to(v.dtype), rem
