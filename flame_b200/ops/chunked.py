"""Chunk-parallel token mixers on the batched tcgen05 GEMM: gated delta rule, delta rule, scalar-gated linear
attention (Mamba2 SSD).

Layout.  Packed tokens ``[T, H, d]`` are re-packed so that every document starts on a chunk boundary (``ChunkLayout``;
chunks of C = 64 or 128 tokens, fewer than C zero rows per document).  In that layout ``[NC, C, H, d]`` every chunk of every head is
one batch of a strided batched GEMM, a zero row contributes nothing (k = v = 0, decay 1), and the whole algorithm
is a short list of batched GEMMs plus elementwise work:

  scores      Akk = strict_tril(beta k k^T e^{b_i-b_j}),  Aqk = tril(scale q k^T e^{b_i-b_j})   (decay + mask in the epilogue)
  WY          T = (I + Akk)^-1,  u = T (beta v),  w = T (beta e^{b} k)
  transition  M_c = khat_c^T w_c,  B_c = khat_c^T u_c          khat = k e^{b_last - b}
  recurrence  S_{c+1} = e^{b_last} S_c - M_c S_c + B_c         one batched GEMM per chunk position, all documents at once
  output      v_new = u - w S,   o = (scale q e^{b}) S + Aqk v_new

The recurrence is the only sequential part; writing the chunk transition as the matrix ``M_c`` turns each step into
a plain GEMM on the state, so it also runs on the batched kernel (state kept in fp32, bf16 mirror as the operand).
The reverse recurrence of the backward pass uses the same launches with ``M_c^T``.

Covers the reference's chunk_gated_delta_rule / chunk_delta_rule / Mamba2 SSD paths
(fla/ops/gated_delta_rule/chunk.py, fla/ops/delta_rule/chunk.py, fla/ops/common/chunk_delta_h.py,
fla/ops/common/chunk_o.py, fla/layers/mamba2.py).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ctypes import c_int, c_longlong, c_void_p

from . import _lib
from .bgemm import MASK_STRICT, MASK_TRIL, _mask, bgemm, bmm
from .varlen import VarlenMeta

CHUNK = 64
_lib.register("fb_gather_rows", [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p])
_lib.register("fb_delta_scan", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p])


# --------------------------------------------------------------------------------------------------------
# recomputation of a token mixer in the backward pass
# --------------------------------------------------------------------------------------------------------
_recompute_mixers = False


def set_mixer_recompute(flag: bool) -> None:
    """With the flag set, the chunk-parallel token mixers below keep only their inputs for the backward pass and run
    their chunk pipeline again there (``--activation_checkpoint.mode selective --activation_checkpoint.selective_ac_option
    mixer``): the pipeline's intermediates - packed operands, WY factors and above all one ``dk x dv`` state per chunk
    and head - are most of what a linear-attention block holds on to (34 GB of states alone for gated_deltanet_1B at
    65,536 tokens), while the projections, norms and the MLP around it are kept as without checkpointing."""
    global _recompute_mixers
    _recompute_mixers = bool(flag)


def _recomputable(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kw):
        if (_recompute_mixers and torch.is_grad_enabled()
                and any(isinstance(a, torch.Tensor) and a.requires_grad for a in args)):
            from torch.utils.checkpoint import checkpoint
            return checkpoint(lambda *t: fn(*t, **kw), *args, use_reentrant=False, preserve_rng_state=False)
        return fn(*args, **kw)
    return wrapper


# --------------------------------------------------------------------------------------------------------
# chunk-aligned layout
# --------------------------------------------------------------------------------------------------------
class ChunkLayout:
    """Where each packed token lives once every document is padded to a multiple of the chunk size."""

    def __init__(self, meta: VarlenMeta, chunk: int = CHUNK) -> None:
        import numpy as np
        lens = np.asarray([n for n in meta.lengths_list() if n > 0], dtype=np.int64)
        dev = meta.device
        self.chunk = chunk
        nchunks = (lens + chunk - 1) // chunk
        self.NC = int(nchunks.sum())
        self.T = int(lens.sum())
        self.Tp = self.NC * chunk
        self.aligned = bool((lens % chunk == 0).all())
        self.n_docs = int(lens.shape[0])
        # built with array operations on the host (a per-token Python loop would sit on the critical path of every step
        # of the linear-attention families): a token's padded row is its packed index plus the padding in front of its
        # document
        first = np.concatenate([[0], np.cumsum(nchunks)[:-1]])
        starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
        rows = np.arange(self.T, dtype=np.int64) + np.repeat(first * chunk - starts, lens)
        last = first + nchunks - 1
        inv = np.full(self.Tp, -1, dtype=np.int32)
        inv[rows] = np.arange(self.T, dtype=np.int32)
        self._first_np, self._nchunks_np = first, nchunks
        self.rows = torch.from_numpy(rows).to(dev)                            # packed token -> padded row
        self.first = torch.from_numpy(first).to(dev)                          # first chunk of every document
        self.last = torch.from_numpy(last).to(dev)                            # last chunk of every document
        self.first_i32, self.last_i32 = self.first.to(torch.int32), self.last.to(torch.int32)
        self.rows_i32 = self.rows.to(torch.int32)
        self.inv_i32 = torch.from_numpy(inv).to(dev)                          # padded row -> packed token, -1 = padding
        self._steps = None

    def _build_steps(self) -> None:
        # chunks at in-document position s that have a successor, and the documents they belong to (only the
        # per-position fallback of the state recurrences walks these)
        import numpy as np
        dev = self.first.device
        docs_all = np.arange(self.n_docs)
        steps, docs = [], []
        for s_ in range(int(self._nchunks_np.max()) - 1 if self.n_docs else 0):
            sel = docs_all[self._nchunks_np > s_ + 1]
            steps.append(torch.from_numpy((self._first_np[sel] + s_).astype(np.int32)).to(dev))
            docs.append(torch.from_numpy(sel.astype(np.int32)).to(dev))
        self._steps, self._step_docs = steps, docs

    @property
    def steps(self):
        if self._steps is None:
            self._build_steps()
        return self._steps

    @property
    def step_docs(self):
        if self._steps is None:
            self._build_steps()
        return self._step_docs

    @staticmethod
    def of(meta: VarlenMeta, chunk: int = CHUNK) -> "ChunkLayout":
        key = ("chunk_layout", chunk)
        lay = meta.cache.get(key)
        if lay is None:
            lay = ChunkLayout(meta, chunk)
            meta.cache[key] = lay
        return lay

    def pack(self, x: torch.Tensor) -> torch.Tensor:
        """[T, ...] -> [NC, chunk, ...] (zero rows where a document is padded)."""
        if self.aligned:
            return x.reshape(self.NC, self.chunk, *x.shape[1:])
        return _Pack.apply(x, self).reshape(self.NC, self.chunk, *x.shape[1:])

    def unpack(self, y: torch.Tensor) -> torch.Tensor:
        """[NC, chunk, ...] -> [T, ...]."""
        y = y.reshape(self.Tp, *y.shape[2:])
        return y if self.aligned else _Unpack.apply(y, self)


def _gather_rows(x: torch.Tensor, idx: torch.Tensor, n_out: int) -> torch.Tensor:
    """``out[r] = x[idx[r]]`` (zero where ``idx[r] < 0``) in one pass of the row-gather kernel."""
    x = x if x.is_contiguous() else x.contiguous()
    row_bytes = (x.numel() // max(x.shape[0], 1)) * x.element_size()
    if not (_lib.available() and x.is_cuda and row_bytes % 16 == 0 and x.shape[0] > 0):
        safe = idx.clamp_min(0).long()
        out = x.index_select(0, safe)
        return out * (idx >= 0).to(x.dtype).view(-1, *([1] * (x.dim() - 1)))
    out = torch.empty(n_out, *x.shape[1:], dtype=x.dtype, device=x.device)
    rc = _lib.lib().fb_gather_rows(x.data_ptr(), out.data_ptr(), idx.data_ptr(), n_out, row_bytes, _lib.stream_ptr())
    _lib.check(rc, "fb_gather_rows")
    _lib.count_launch()
    return out


class _Pack(torch.autograd.Function):
    """Packed rows into the padded layout (zero rows where a document is padded): a gather through the inverse row map;
    the map is injective, so the backward is a plain gather too."""

    @staticmethod
    def forward(ctx, x, lay):
        ctx.lay = lay
        return _gather_rows(x, lay.inv_i32, lay.Tp)

    @staticmethod
    def backward(ctx, dy):
        return _gather_rows(dy, ctx.lay.rows_i32, ctx.lay.T), None


class _Unpack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, lay):
        ctx.lay = lay
        return _gather_rows(y, lay.rows_i32, lay.T)

    @staticmethod
    def backward(ctx, dx):
        return _gather_rows(dx, ctx.lay.inv_i32, ctx.lay.Tp), None


def _hm(x: torch.Tensor) -> torch.Tensor:
    """[NC, 64, H, d] -> the [NC, H, 64, d] operand view."""
    return x.permute(0, 2, 1, 3)


# --------------------------------------------------------------------------------------------------------
# differentiable pieces
# --------------------------------------------------------------------------------------------------------
class _Scores(torch.autograd.Function):
    """``C = mask(alpha * A B^T * exp(d_i - d_j))`` for 64 x 64 score blocks; ``d`` is the within-chunk cumulative log decay."""

    @staticmethod
    def forward(ctx, a, b, d, alpha, mask, out_dtype):
        # a, b: [NC, G, C, dk] views (G heads, G divides H); d: [NC, H, C] fp32: one score block per head from shared q / k
        out = bgemm(a, b, alpha=alpha, mask=mask, decay=d, out_dtype=out_dtype, n_lo=d.shape[1])
        ctx.save_for_backward(a, b, d, out)
        ctx.cfg = (alpha, mask)
        return out

    @staticmethod
    def backward(ctx, dc):
        a, b, d, out = ctx.saved_tensors
        alpha, mask = ctx.cfg
        C = out.shape[-1]
        if _lib.available() and out.is_cuda and out.dtype in (torch.float32, torch.bfloat16) and C % 32 == 0 and C <= 128 \
                and d.dtype == torch.float32:
            from . import chunk_kernels
            g, dd = chunk_kernels.scores_bwd_prep(dc, out, d, mask)       # one pass instead of eight elementwise ones
        else:
            dcf = dc.float()
            dd = None
            if ctx.needs_input_grad[2]:
                e = dcf * out.float()
                dd = e.sum(-1) - e.sum(-2)
            m = _mask(out.shape[-2], out.shape[-1], mask, dc.device)
            w = (d[..., :, None] - d[..., None, :]).masked_fill(~m, float("-inf")).exp()
            g = dcf * w
        NC, H = g.shape[:2]
        G = a.shape[1]
        if G < H:  # shared q / k: the heads of a group add up on the (small) score gradient before the GEMMs
            g = g.reshape(NC, G, H // G, *g.shape[2:]).float().sum(2)
        g = g.to(a.dtype)
        da = db = None
        if ctx.needs_input_grad[0]:
            da = _like(a)
            bgemm(g, b, b_mn=True, out=da, alpha=alpha)
        if ctx.needs_input_grad[1]:
            db = _like(b)
            bgemm(g, a, a_mn=True, b_mn=True, out=db, alpha=alpha)
        return da, db, dd, None, None, None


def _like(t: torch.Tensor) -> torch.Tensor:
    from .bgemm import _empty_like_layout
    return _empty_like_layout(t)


def tri_inverse(A: torch.Tensor) -> torch.Tensor:
    """``(I + A)^-1`` for strictly lower-triangular ``A [NC, H, n, n]`` (fp32), n = 64 or 128, no autograd.
    n = 128 is inverted blockwise: with A = [[A11, 0], [A21, A22]] the inverse is [[T11, 0], [-T22 A21 T11, T22]]
    where T11, T22 come from the 64 x 64 kernel and the corner from two batched GEMMs."""
    n = A.shape[-1]
    if _lib.available() and A.is_cuda:
        from . import chunk_kernels
        if n == 64:
            return chunk_kernels.tri_inverse(A, torch.bfloat16)
        assert n == 128, "chunk sizes 64 and 128 are supported"
        h = 64
        diag = torch.stack((A[..., :h, :h], A[..., h:, h:]), 0).contiguous()
        Td = chunk_kernels.tri_inverse(diag, torch.bfloat16)            # [2, NC, H, 64, 64]
        T11, T22 = Td[0], Td[1]
        X = bgemm(T22, A[..., h:, :h].to(torch.bfloat16), b_mn=True)     # T22 A21
        out = torch.zeros(A.shape, dtype=torch.bfloat16, device=A.device)
        out[..., :h, :h] = T11
        out[..., h:, h:] = T22
        bgemm(X, T11, b_mn=True, alpha=-1.0, out=out[..., h:, :h])
        return out
    eye = torch.eye(n, dtype=torch.float32, device=A.device)
    return torch.linalg.solve_triangular(eye + A.float(), eye.expand_as(A).contiguous(), upper=False, unitriangular=True)


class _TriInv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A):
        T = tri_inverse(A).to(torch.bfloat16 if A.is_cuda else A.dtype).contiguous()
        ctx.save_for_backward(T)
        return T

    @staticmethod
    def backward(ctx, dT):
        (T,) = ctx.saved_tensors
        dT = dT.to(T.dtype)
        # dA = -T^T dT T^T, kept on the strict lower triangle
        x = bgemm(T, dT, a_mn=True, b_mn=True)
        dA = bgemm(x, T, alpha=-1.0, mask=MASK_STRICT, out_dtype=torch.float32)
        return dA


class _DeltaScan(torch.autograd.Function):
    """States at the start of every chunk for ``S_{c+1} = alpha_c S_c - (khat_c^T w_c) S_c + khat_c^T u_c`` (S = 0 at
    the first chunk of a document).  ``w = None`` drops the middle term (plain gated linear attention); then ``alpha``
    may also be ``[NC, H, dk]`` (one decay per key channel).

    With ``w`` the running state lives in ONE fp32 buffer per document (``[docs, H, dk, dv]``, updated in place by the
    GEMM epilogue and small enough to stay in L2); only its bf16 copy is written per chunk."""

    @staticmethod
    def forward(ctx, alpha, khat, w, u, lay: ChunkLayout):
        # alpha [NC, H] fp32; khat, w [NC, H, C, dk]; u [NC, H, C, dv] (operand views); without w, khat may have fewer
        # heads than u (keys shared by groups of heads)
        NC, _, _, dk = khat.shape
        H = u.shape[1]
        dv = u.shape[-1]
        dev = khat.device
        alpha = alpha.contiguous()
        S16 = torch.empty(NC + 1, H, dk, dv, dtype=khat.dtype, device=dev)
        S16.index_fill_(0, lay.first, 0.0)
        if w is not None:
            M = bgemm(khat, w, a_mn=True, b_mn=True)                 # [NC, H, dk, dk] chunk transition
            B16 = bgemm(khat, u, a_mn=True, b_mn=True)               # [NC, H, dk, dv] chunk increment
            if _scan_kernel_ok(M, B16, alpha, dk, dv):
                _delta_scan(M, B16, alpha, S16, lay, reverse=False)   # one persistent launch walks every document
            else:  # shapes the scan kernel does not cover: one batched GEMM per chunk position
                state = torch.zeros(lay.n_docs, H, dk, dv, dtype=torch.float32, device=dev)
                for idx, docs in zip(lay.steps, lay.step_docs):
                    bgemm(M, S16, b_mn=True, a_index=idx, b_index=idx, out=state, c_index=docs, cin=state,
                          cin_index=docs, gamma=alpha, alpha=-1.0, add16=B16, add16_index=idx, out16=S16,
                          out16_index=idx, out16_offset=1, n_hi=len(idx))
        else:
            M = None
            Sf = torch.empty(NC + 1, H, dk, dv, dtype=torch.float32, device=dev)
            bgemm(khat, u, a_mn=True, b_mn=True, out=Sf, c_offset=1)
            Sf.index_fill_(0, lay.first, 0.0)
            _elementwise_steps(lay, alpha, Sf, S16, reverse=False)
        ctx.save_for_backward(alpha, khat, w, u, M, S16)
        ctx.lay = lay
        return S16[:NC]

    @staticmethod
    def backward(ctx, dS):
        alpha, khat, w, u, M, S16 = ctx.saved_tensors
        lay = ctx.lay
        NC, _, _, dk = khat.shape
        H = u.shape[1]
        dv = u.shape[-1]
        dev = khat.device
        dS = dS.to(khat.dtype).contiguous()
        L16 = torch.empty(NC + 1, H, dk, dv, dtype=khat.dtype, device=dev)
        L16[:NC] = dS
        L16[NC] = 0
        if M is not None and _scan_kernel_ok(M, dS, alpha, dk, dv):
            _delta_scan(M, dS, alpha, L16, lay, reverse=True)
        elif M is not None:
            # adjoint state per document, started from the gradient of the document's last chunk state
            lam = dS.index_select(0, lay.last).float()
            for idx, docs in zip(lay.steps[::-1], lay.step_docs[::-1]):
                bgemm(M, L16, a_mn=True, b_mn=True, a_index=idx, b_index=idx, b_offset=1, out=lam, c_index=docs, cin=lam,
                      cin_index=docs, gamma=alpha, alpha=-1.0, add16=dS, add16_index=idx, out16=L16, out16_index=idx,
                      n_hi=len(idx))
        else:
            Lf = torch.empty(NC + 1, H, dk, dv, dtype=torch.float32, device=dev)
            Lf[:NC] = dS
            Lf[NC] = 0
            _elementwise_steps(lay, alpha, Lf, L16, reverse=True)
        # adjoint of the state entering the NEXT chunk; zero where the next chunk belongs to another document
        L16.index_fill_(0, lay.first, 0.0)
        Ln = L16[1:]
        S = S16[:NC]
        dalpha = dkhat = dw = du = None
        if ctx.needs_input_grad[0]:
            dalpha = _pair_dot(Ln, S, per_row=alpha.dim() == 3)
        # B_c = khat^T u
        dkh = bgemm(u, Ln, out_dtype=torch.float32, out=_token_major(NC, H, lay.chunk, dk, torch.float32, dev))
        if ctx.needs_input_grad[3]:
            du = _like(u)
            bgemm(khat, Ln, b_mn=True, out=du)
        if w is not None:
            dM = bgemm(Ln, S, alpha=-1.0)  # [NC, H, dk, dk]
            bgemm(w, dM, out=dkh, accumulate=True)
            if ctx.needs_input_grad[2]:
                dw = _like(w)
                bgemm(khat, dM, b_mn=True, out=dw)
        if ctx.needs_input_grad[1]:
            G = khat.shape[1]
            if G < H:  # keys shared by the heads of a group
                dkh = dkh.reshape(NC, G, H // G, *dkh.shape[2:]).sum(2)
            dkhat = dkh.to(khat.dtype)
        return dalpha, dkhat, dw, du, None


def _scan_kernel_ok(M: torch.Tensor, add: torch.Tensor, alpha: torch.Tensor, dk: int, dv: int) -> bool:
    import os
    return (_lib.available() and M.is_cuda and M.dtype == torch.bfloat16 and add.dtype == torch.bfloat16
            and M.is_contiguous() and add.is_contiguous() and alpha.dim() == 2 and alpha.dtype == torch.float32
            and dk in (128, 256) and dv % 128 == 0 and os.environ.get("FLAME_B200_DELTA_SCAN", "1") != "0")


def _delta_scan(M: torch.Tensor, add: torch.Tensor, alpha: torch.Tensor, out16: torch.Tensor, lay: "ChunkLayout",
                reverse: bool) -> None:
    """The chunk-state recurrence of every (document, head) in one persistent kernel (``csrc/delta_scan.cu``)."""
    NC, H, dk, _ = M.shape
    dv = add.shape[-1]
    first, last = lay.first_i32, lay.last_i32
    rc = _lib.lib().fb_delta_scan(M.data_ptr(), add.data_ptr(), alpha.data_ptr(), out16.data_ptr(), first.data_ptr(),
                                  last.data_ptr(), lay.n_docs, H, NC, dk, dv, 1 if reverse else 0, _lib.stream_ptr())
    _lib.check(rc, "fb_delta_scan")
    _lib.count_launch()


def _pair_dot(x: torch.Tensor, y: torch.Tensor, per_row: bool) -> torch.Tensor:
    """``sum(x * y)`` over the last two (or the last) dimensions in fp32 without materialising fp32 copies."""
    if _lib.available() and x.is_cuda:
        from . import chunk_kernels
        return chunk_kernels.pair_dot(x, y, per_row)
    return (x.float() * y.float()).sum(-1 if per_row else (-1, -2))


def _token_major(NC, H, R, D, dtype, dev):
    return torch.empty(NC, R, H, D, dtype=dtype, device=dev).permute(0, 2, 1, 3)


def _elementwise_steps(lay: ChunkLayout, alpha, Xf, X16, reverse: bool) -> None:
    """Forward: X[c+1] = alpha_c X[c] + X[c+1].  Reverse: X[c] = alpha_c X[c+1] + X[c] (fp32, bf16 mirror)."""
    if _lib.available() and Xf.is_cuda:
        from . import chunk_kernels
        chunk_kernels.state_scan(lay.first, lay.last, alpha, Xf, X16, reverse)
        return
    steps = lay.steps[::-1] if reverse else lay.steps
    for idx in steps:
        i = idx.long()
        src, dst = (i + 1, i) if reverse else (i, i + 1)
        al = alpha[i][..., None] if alpha.dim() == 3 else alpha[i][..., None, None]
        r = Xf[dst] + al * Xf[src]
        Xf[dst] = r
        X16[dst] = r.to(X16.dtype)


# --------------------------------------------------------------------------------------------------------
# algorithms
# --------------------------------------------------------------------------------------------------------
def _scalar_prep(qp, kp, gp, scale, dt):
    """``b = cumsum(g)`` [NC, C, H], ``khat = k e^{b_last - b}``, ``qbar = scale q e^{b}``, ``alpha = e^{b_last}`` [NC, H]."""
    NC, C, H, dk = qp.shape
    if _lib.available() and qp.is_cuda:
        from . import chunk_kernels
        if chunk_kernels.scalar_prep_supported(C, dk):
            return chunk_kernels.ScalarPrep.apply(qp, kp, gp, scale)
    b = gp.cumsum(1) if gp is not None else torch.zeros(NC, C, H, dtype=torch.float32, device=qp.device)
    b_last = b[:, -1]
    khat = kp * (b_last[:, None] - b).exp().to(dt)[..., None]
    qbar = qp * (b.exp() * scale).to(dt)[..., None]
    return b, khat, qbar, b_last.exp()


def scalar_chunk(dk: int, dv: int) -> int:
    """Chunk length of the scalar-gated algorithms.  With a large state (dk * dv) 128 halves the number of sequential
    state steps and of stored chunk states and fills the 128-row MMA tile; with a small state the 64 x 64 score blocks
    are the cheaper side.  Every decay exponent stays <= 0 at any chunk length."""
    return 128 if dk * dv >= 32768 else 64


@_recomputable
def gated_delta_rule_tc(q, k, v, beta, g, meta: VarlenMeta, scale: Optional[float] = None,
                        chunk: Optional[int] = None) -> torch.Tensor:
    """Chunked (gated) delta rule; q, k ``[T, H, dk]`` (already normalised), v ``[T, H, dv]``, beta ``[T, H]``,
    g ``[T, H]`` log decay or None.  Same result as ``linear_attn.gated_delta_rule_recurrent``."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    lay = ChunkLayout.of(meta, chunk or scalar_chunk(dk, dv))
    dt = torch.bfloat16 if q.is_cuda else q.dtype
    qp, kp, vp = lay.pack(q).to(dt), lay.pack(k).to(dt), lay.pack(v).to(dt)   # [NC, C, H, d]
    bp = lay.pack(beta.float())                                      # [NC, C, H]
    # the only token-sized derived operands: khat = k e^{b_last - b} and qbar = scale q e^{b}; every other scaling
    # (beta, beta e^{b}) is folded into the C x C matrices
    b, khat, qbar, alpha = _scalar_prep(qp, kp, None if g is None else lay.pack(g.float()), scale, dt)
    d = b.permute(0, 2, 1)                                           # [NC, H, 64] view
    beta_r = bp.permute(0, 2, 1)                                     # [NC, H, 64]
    Akk = _Scores.apply(_hm(kp), _hm(kp), d, 1.0, MASK_STRICT, torch.float32) * beta_r[..., None]
    Aqk = _Scores.apply(_hm(qp), _hm(kp), d, scale, MASK_TRIL, dt)
    Tm = _TriInv.apply(Akk)                                          # [NC, H, 64, 64]
    Tu = Tm * beta_r.to(dt)[..., None, :]
    Tw = Tm * (beta_r * d.exp()).to(dt)[..., None, :]
    u = bmm(Tu, _hm(vp), b_mn=True, token_major=True, out_dtype=dt)  # [NC, H, 64, dv] view of [NC, 64, H, dv]
    w = bmm(Tw, _hm(kp), b_mn=True, token_major=True, out_dtype=dt)
    S = _DeltaScan.apply(alpha, _hm(khat), w, u, lay)                # [NC, H, dk, dv]
    v_new = bmm(w, S, b_mn=True, token_major=True, out_dtype=dt, alpha=-1.0, addend=u)      # u - w S
    o = bmm(_hm(qbar), S, b_mn=True, token_major=True, out_dtype=dt)
    o = bmm(Aqk, v_new, b_mn=True, token_major=True, out_dtype=dt, addend=o)
    return lay.unpack(o.permute(0, 2, 1, 3)).to(v.dtype)


@_recomputable
def scalar_gla_tc(q, k, v, g, meta: VarlenMeta, scale: float = 1.0, chunk: Optional[int] = None) -> torch.Tensor:
    """``S_t = exp(g_t) S_{t-1} + k_t v_t^T,  o_t = scale q_t^T S_t`` with one log decay per head and step
    (Mamba2's SSD in its attention form).  q, k ``[T, G, dk]`` with G dividing H, v ``[T, H, dv]``, g ``[T, H]``."""
    T, G, dk = q.shape
    H = v.shape[1]
    lay = ChunkLayout.of(meta, chunk or scalar_chunk(dk, v.shape[-1]))
    dt = torch.bfloat16 if q.is_cuda else q.dtype
    qp, kp, vp = lay.pack(q).to(dt), lay.pack(k).to(dt), lay.pack(v).to(dt)
    if G < H:
        # q and k are shared by groups of H / G heads (Mamba2's B and C): they are never expanded.  The decay moves to the
        # value side of the state update (S += k^T (v e^{b_last - b})) and to the rows of the inter-chunk output.
        b = lay.pack(g.float()).cumsum(1)                              # [NC, C, H]
        b_last = b[:, -1]
        vhat = vp * (b_last[:, None] - b).exp().to(dt)[..., None]
        d = b.permute(0, 2, 1)
        Aqk = _Scores.apply(_hm(qp), _hm(kp), d, scale, MASK_TRIL, dt)  # [NC, H, C, C] from the G shared q / k
        S = _DeltaScan.apply(b_last.exp(), _hm(kp), None, _hm(vhat), lay)
        o = bmm(_hm(qp), S, b_mn=True, token_major=True, out_dtype=dt) * (b.exp() * scale).to(dt).permute(0, 2, 1)[..., None]
        o = bmm(Aqk, _hm(vp), b_mn=True, token_major=True, out_dtype=dt, addend=o)
        return lay.unpack(o.permute(0, 2, 1, 3)).to(v.dtype)
    b, khat, qbar, alpha = _scalar_prep(qp, kp, lay.pack(g.float()), scale, dt)
    d = b.permute(0, 2, 1)
    Aqk = _Scores.apply(_hm(qp), _hm(kp), d, scale, MASK_TRIL, dt)
    S = _DeltaScan.apply(alpha, _hm(khat), None, _hm(vp), lay)
    o = bmm(_hm(qbar), S, b_mn=True, token_major=True, out_dtype=dt)
    o = bmm(Aqk, _hm(vp), b_mn=True, token_major=True, out_dtype=dt, addend=o)
    return lay.unpack(o.permute(0, 2, 1, 3)).to(v.dtype)


class _GlaDiag(torch.autograd.Function):
    """Diagonal 16 x 16 sub-blocks of the GLA intra-chunk scores (exact pairwise exponents) on the CUDA kernel."""

    @staticmethod
    def forward(ctx, qp, kp, b, scale):
        from . import chunk_kernels
        NC, C, H, dk = qp.shape
        A = torch.zeros(NC, H, C, C, dtype=torch.float32, device=qp.device)
        qp, kp, b = qp.contiguous(), kp.contiguous(), b.contiguous()
        chunk_kernels.gla_diag_fwd(qp, kp, b, scale, A)
        ctx.save_for_backward(qp, kp, b)
        ctx.scale = scale
        return A

    @staticmethod
    def backward(ctx, dA):
        from . import chunk_kernels
        qp, kp, b = ctx.saved_tensors
        dq = torch.zeros(qp.shape, dtype=torch.float32, device=qp.device)
        dk = torch.zeros_like(dq)
        db = torch.zeros_like(dq)
        chunk_kernels.gla_diag_bwd(qp, kp, b, dA.float().contiguous(), dq, dk, db, ctx.scale)
        return dq.to(qp.dtype), dk.to(kp.dtype), db, None


def _gla_diag(qp, kp, b, scale, sub: int = 16):
    """[NC, H, 64, 64] fp32 holding only the diagonal sub-blocks of A_ij = scale sum_d q_id k_jd exp(b_id - b_jd), j <= i."""
    if _lib.available() and qp.is_cuda:
        return _GlaDiag.apply(qp, kp, b, scale)
    NC, C, H, dk = qp.shape
    A = torch.zeros(NC, H, C, C, dtype=torch.float32, device=qp.device)
    tri = torch.tril(torch.ones(sub, sub, dtype=torch.bool, device=qp.device))
    for i in range(C // sub):
        rows = slice(i * sub, (i + 1) * sub)
        d = b[:, rows, None] - b[:, None, rows]                       # [NC, sub, sub, H, dk]
        d = d.masked_fill(~tri[None, :, :, None, None], float("-inf")).exp()
        A[:, :, rows, rows] = torch.einsum("nihd,njhd,nijhd->nhij", qp[:, rows].float(), kp[:, rows].float(), d) * scale
    return A


@_recomputable
def gla_tc(q, k, v, g, meta: VarlenMeta, scale: Optional[float] = None, sub: int = 16) -> torch.Tensor:
    """Chunked gated linear attention with one log decay per key channel: q, k, g ``[T, H, dk]``, v ``[T, H, dv]``.
    Same result as ``linear_attn.gla_recurrent``.  Inside a chunk the scores are built from 16-row sub-blocks:
    off-diagonal sub-blocks as products re-based on the query sub-block's first row (batched GEMM), diagonal
    sub-blocks pairwise, so every exponent is <= 0 for any gate values (fla/ops/gla/chunk.py:88-170)."""
    T, H, dk = q.shape
    scale = dk ** -0.5 if scale is None else scale
    lay = ChunkLayout.of(meta)
    dt = torch.bfloat16 if q.is_cuda else q.dtype
    qp, kp, vp = lay.pack(q).to(dt), lay.pack(k).to(dt), lay.pack(v).to(dt)   # [NC, 64, H, d]
    C = lay.chunk
    nb = C // sub
    NC = qp.shape[0]
    ncol = C - sub
    if _lib.available() and q.is_cuda and C == 64 and sub == 16:
        # cumulative decay and every scaled operand in one kernel (and one for the whole backward of this stage)
        from .chunk_kernels import GlaPrep
        b, khat, qbar, qt, k3, alpha = GlaPrep.apply(qp, kp, lay.pack(g.float()), scale)
    else:
        b = lay.pack(g.float()).cumsum(1)                                      # [NC, 64, H, dk]
        b_last = b[:, -1]                                                      # [NC, H, dk]
        alpha = b_last.exp()
        khat = kp * (b_last[:, None] - b).exp().to(dt)
        qbar = qp * (b.exp() * scale).to(dt)
        # off-diagonal sub-blocks: batch (chunk, I) multiplies the 16 query rows of sub-block I, re-based on the
        # sub-block's first row, with the keys before it re-based on the same row; later keys are zeroed
        r = b[:, ::sub].detach()                                               # [NC, nb, H, dk]
        qt = qp * (b - r.repeat_interleave(sub, 1)).exp().to(dt)
        expo = r[:, 1:, None] - b[:, None, :ncol]                              # [NC, nb-1, ncol, H, dk]
        keep = (torch.arange(ncol, device=q.device)[None, :] < (torch.arange(1, nb, device=q.device) * sub)[:, None])
        keep = keep[None, :, :, None, None]
        k3 = (kp[:, None, :ncol] * torch.where(keep, expo, expo.new_full((), float("-inf"))).exp().to(dt))
    S = _DeltaScan.apply(alpha, _hm(khat), None, _hm(vp), lay)                 # [NC, H, dk, dv]
    o = bmm(_hm(qbar), S, b_mn=True, token_major=True, out_dtype=dt)
    A = _gla_diag(qp, kp, b, scale, sub)
    # all off-diagonal sub-blocks in ONE batched GEMM
    qt3 = qt[:, sub:].reshape(NC * (nb - 1), sub, H, dk)
    k3 = k3.reshape(NC * (nb - 1), ncol, H, dk)
    blk = bmm(_hm(qt3), _hm(k3), alpha=scale, out_dtype=torch.float32)         # [NC*(nb-1), H, sub, ncol]
    blk = blk.reshape(NC, nb - 1, H, sub, ncol).permute(0, 2, 1, 3, 4).reshape(NC, H, C - sub, ncol)
    A = A + torch.nn.functional.pad(blk, (0, sub, sub, 0))
    o = bmm(A.to(dt), _hm(vp), b_mn=True, token_major=True, out_dtype=dt, addend=o)
    return lay.unpack(o.permute(0, 2, 1, 3)).to(v.dtype)


@_recomputable
def gla_vdecay_tc(q, k, v, gv, meta: VarlenMeta, scale: float, sub: int = 16) -> torch.Tensor:
    """``S_t = S_{t-1} diag(exp gv_t) + k_t v_t^T,  o_t = scale q_t^T S_t``: the state decays along its VALUE dimension
    (first pass of gated slot attention, fla/ops/gsa/chunk.py).  q, k ``[T, H, dk]``, v, gv ``[T, H, dv]``; returns fp32.
    The state is carried transposed (``[dv, dk]``) so that the decay is per state row like in ``gla_tc``."""
    T, H, dk = q.shape
    lay = ChunkLayout.of(meta)
    dt = torch.bfloat16 if q.is_cuda else q.dtype
    C = lay.chunk
    qp, kp, vp = lay.pack(q).to(dt), lay.pack(k).to(dt), lay.pack(v).to(dt)
    b = lay.pack(gv.float()).cumsum(1)                                         # [NC, 64, H, dv]
    b_last = b[:, -1]
    vhat = vp * (b_last[:, None] - b).exp().to(dt)
    St = _DeltaScan.apply(b_last.exp(), _hm(vhat), None, _hm(kp), lay)         # [NC, H, dv, dk]
    o = bmm(_hm(qp), St, token_major=True, out_dtype=torch.float32).permute(0, 2, 1, 3) * b.exp()   # [NC, 64, H, dv]
    P = bgemm_scores_plain(qp, kp)                                             # [NC, H, 64, 64] tril(q k^T)
    use_kernel = _lib.available() and q.is_cuda and C == 64 and sub == 16
    nb, ncol, NC = C // sub, C - sub, qp.shape[0]
    dv = vp.shape[-1]
    # off-diagonal sub-blocks, all in ONE batched GEMM: batch (chunk, I) multiplies the 16 score rows of sub-block I with
    # the values before it, re-based on the sub-block's first row r_I (every exponent is <= 0); values from sub-block I
    # on are zeroed, so the product may run over all 48 columns
    r = b[:, ::sub].detach()                                                   # [NC, nb, H, dv]
    expo = r[:, 1:, None] - b[:, None, :ncol]                                  # [NC, nb-1, ncol, H, dv]
    keep = (torch.arange(ncol, device=q.device)[None, :] < (torch.arange(1, nb, device=q.device) * sub)[:, None])
    keep = keep[None, :, :, None, None]
    v3 = vp[:, None, :ncol] * torch.where(keep, expo, expo.new_full((), float("-inf"))).exp().to(dt)
    P3 = P[:, :, sub:, :ncol].reshape(NC, H, nb - 1, sub, ncol).permute(0, 2, 1, 3, 4).reshape(NC * (nb - 1), H, sub, ncol)
    acc = bmm(P3.to(dt), _hm(v3.reshape(NC * (nb - 1), ncol, H, dv)), b_mn=True, token_major=True,
              out_dtype=torch.float32)                                         # [NC*(nb-1), H, sub, dv] over [.., sub, H, dv]
    acc = acc.permute(0, 2, 1, 3).reshape(NC, ncol, H, dv) * (b[:, sub:] - r[:, 1:].repeat_interleave(sub, 1)).exp()
    o = o + torch.nn.functional.pad(acc, (0, 0, 0, 0, sub, 0))
    if use_kernel:
        from .chunk_kernels import VdecayDiag
        o = o + VdecayDiag.apply(P, vp, b)                                     # all diagonal sub-blocks, exact
    else:
        tri = torch.tril(torch.ones(sub, sub, dtype=torch.bool, device=q.device))
        parts = []
        for i in range(nb):
            rows = slice(i * sub, (i + 1) * sub)
            dd = (b[:, rows, None] - b[:, None, rows]).masked_fill(~tri[None, :, :, None, None], float("-inf")).exp()
            parts.append(torch.einsum("nhij,njhc,nijhc->nihc", P[:, :, rows, rows].float(), vp[:, rows].float(), dd))
        o = o + torch.cat(parts, 1)
    o = o * scale
    return lay.unpack(o)


def bgemm_scores_plain(qp, kp):
    """``tril(q k^T)`` per chunk and head, differentiable: [NC, H, 64, 64] fp32."""
    zero = torch.zeros(qp.shape[0], qp.shape[2], qp.shape[1], dtype=torch.float32, device=qp.device)
    return _Scores.apply(_hm(qp), _hm(kp), zero, 1.0, MASK_TRIL, torch.float32)
