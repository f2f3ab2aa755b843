"""sm_100a batched GEMM and chunk-algorithm kernels against PyTorch fp32 oracles (needs a B200: ``pytest -m gpu``)."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    from flame_b200.ops import _lib
    _lib.lib()
    _lib.status_clear()
    yield
    torch.cuda.synchronize()
    assert _lib.status() == 0, f"kernel status word {_lib.status():#x}"


def _meta(lens):
    from flame_b200.ops.varlen import VarlenMeta
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return VarlenMeta.from_cu_seqlens(cu, sum(lens), torch.device(DEV))


def _bf(*shape, s=0.5):
    return (torch.randn(*shape, device=DEV) * s).to(torch.bfloat16)


def _ref(a, b, a_mn, b_mn):
    af = a.float().transpose(-1, -2) if a_mn else a.float()
    bf = b.float() if b_mn else b.float().transpose(-1, -2)
    return af @ bf


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_bgemm_layouts_on_chunk_views(a_mn, b_mn):
    from flame_b200.ops.bgemm import bgemm
    torch.manual_seed(0)
    NC, H, M, N, K = 19, 3, 64, 256, 128
    # operands are permuted views of token-major storage, as the chunk algorithms pass them
    a = _bf(NC, K if a_mn else M, H, M if a_mn else K).permute(0, 2, 1, 3)
    b = _bf(NC, K if b_mn else N, H, N if b_mn else K).permute(0, 2, 1, 3)
    out = bgemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert rel_err(out, _ref(a, b, a_mn, b_mn)) < 1e-5 + 3e-3
    out16 = torch.empty(NC, M, H, N, device=DEV, dtype=torch.bfloat16).permute(0, 2, 1, 3)
    bgemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out16, alpha=0.5)
    assert rel_err(out16, 0.5 * _ref(a, b, a_mn, b_mn)) < 1e-2


def test_bgemm_mask_decay_and_state_step():
    from flame_b200.ops.bgemm import MASK_STRICT, MASK_TRIL, bgemm
    torch.manual_seed(1)
    NC, H, dk, dv = 11, 2, 128, 256
    q, k = _bf(NC, 64, H, dk).permute(0, 2, 1, 3), _bf(NC, 64, H, dk).permute(0, 2, 1, 3)
    d = (-torch.rand(NC, 64, H, device=DEV) * 0.3).cumsum(1).permute(0, 2, 1)
    full = (q.float() @ k.float().transpose(-1, -2)) * (d[..., :, None] - d[..., None, :]).exp()
    assert rel_err(bgemm(q, k, decay=d, mask=MASK_TRIL, out_dtype=torch.float32), full.tril()) < 5e-3
    assert rel_err(bgemm(q, k, decay=d, mask=MASK_STRICT, alpha=0.25), 0.25 * full.tril(-1)) < 1e-2
    # state step through index tables: X[c+1] = gamma_c X[c] - M_c X16[c] + X[c+1]
    M = _bf(NC, H, dk, dk, s=0.05)
    Xf = torch.randn(NC + 1, H, dk, dv, device=DEV)
    X16 = Xf.to(torch.bfloat16)
    gam = torch.rand(NC, H, device=DEV)
    idx = torch.tensor([0, 2, 5, 9], device=DEV, dtype=torch.int32)
    i = idx.long()
    want = Xf.clone()
    want[i + 1] = Xf[i + 1] + gam[i][..., None, None] * Xf[i] - M[i].float() @ X16[i].float()
    bgemm(M, X16, b_mn=True, a_index=idx, b_index=idx, out=Xf, c_index=idx, c_offset=1, accumulate=True, cin=Xf,
          cin_index=idx, gamma=gam, alpha=-1.0, out16=X16, out16_index=idx, out16_offset=1, n_hi=len(idx))
    assert rel_err(Xf, want) < 1e-3
    assert rel_err(X16, want) < 1e-2
    # in-place per-document state: state[d] = gamma_c state[d] - M_c X16[c] + add16[c], bf16 copy to X16[c+1]
    docs = torch.tensor([3, 0, 2, 1], device=DEV, dtype=torch.int32)
    state = torch.randn(4, H, dk, dv, device=DEV)
    add = _bf(NC, H, dk, dv)
    X16 = want.to(torch.bfloat16)
    want_state = state.clone()
    want_state[docs.long()] = gam[i][..., None, None] * state[docs.long()] - M[i].float() @ X16[i].float() + add[i].float()
    want16 = X16.clone()
    want16[i + 1] = want_state[docs.long()].to(torch.bfloat16)
    bgemm(M, X16, b_mn=True, a_index=idx, b_index=idx, out=state, c_index=docs, cin=state, cin_index=docs, gamma=gam,
          alpha=-1.0, add16=add, add16_index=idx, out16=X16, out16_index=idx, out16_offset=1, n_hi=len(idx))
    assert rel_err(state, want_state) < 1e-3
    assert rel_err(X16, want16) < 1e-2


def test_tri_inverse_and_l2norm():
    from flame_b200.ops.chunk_kernels import l2norm, tri_inverse
    torch.manual_seed(2)
    A = (torch.randn(7, 3, 64, 64, device=DEV) * 0.2).tril(-1)
    eye = torch.eye(64, device=DEV)
    ref = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False, unitriangular=True)
    assert rel_err(tri_inverse(A, torch.float32), ref) < 1e-5
    x = torch.randn(1000, 6, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = l2norm(x)
    xf = x.detach().float().requires_grad_(True)
    yr = xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + 1e-6)
    assert rel_err(y, yr) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    assert rel_err(x.grad, xf.grad) < 2e-2


def _run(fn, inputs, f32):
    for t in inputs:
        t.grad = None
    o = fn((lambda x: x.float()) if f32 else (lambda x: x))
    torch.manual_seed(99)
    (o.float() * torch.randn(o.shape, device=DEV)).sum().backward()
    return [o.detach()] + [t.grad.clone() for t in inputs]


LENS = [300, 77, 129, 64, 1000, 1]


@pytest.mark.parametrize("gated,chunk,dk,dv", [(True, 128, 128, 256), (False, 128, 128, 256), (True, 64, 128, 256),
                                                 (True, 128, 256, 128), (False, 64, 128, 128), (True, 64, 64, 64)])
def test_gated_delta_rule_kernels_match_fp32_chunk_reference(gated, chunk, dk, dv):
    """dk 128 / 256 with dv a multiple of 128 walk the chunk states in the persistent scan kernel (csrc/delta_scan.cu);
    the last case takes the one-launch-per-position path."""
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.chunked import gated_delta_rule_tc
    torch.manual_seed(3)
    meta = _meta(LENS)
    T, H = sum(LENS), 2
    leaf = lambda *s: torch.randn(*s, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    q, k, v, braw, graw = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv), leaf(T, H), leaf(T, H)
    ins = [q, k, v, braw] + ([graw] if gated else [])

    def make(fn):
        def f(c):
            g = -F.softplus(graw.float()) * 0.3 if gated else None
            return fn(la.l2norm(c(q)), la.l2norm(c(k)), c(v), braw.float().sigmoid(), g, meta)
        return f
    ref = _run(make(la.gated_delta_rule_chunk), ins, True)
    out = _run(make(lambda *a: gated_delta_rule_tc(*a, chunk=chunk)), ins, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 3e-2


def test_delta_scan_kernel_equals_the_per_position_launches(monkeypatch):
    """Same chunk states, bit for bit, from the persistent scan kernel and from one batched GEMM per chunk position
    (both keep the state in fp32 and feed its bf16 rounding to the tensor core), forward and reverse."""
    from flame_b200.ops import chunked
    from flame_b200.ops.bgemm import bgemm
    torch.manual_seed(5)
    lay = chunked.ChunkLayout.of(_meta([700, 64, 129, 2000]), 64)
    NC, H, dk, dv = lay.NC, 3, 128, 256
    M = (torch.randn(NC, H, dk, dk, device=DEV) * 0.05).to(torch.bfloat16)
    B = torch.randn(NC, H, dk, dv, device=DEV).to(torch.bfloat16)
    alpha = torch.rand(NC, H, device=DEV) * 0.5 + 0.5
    outs = []
    for use_scan in (True, False):
        S16 = torch.empty(NC + 1, H, dk, dv, dtype=torch.bfloat16, device=DEV)
        S16.index_fill_(0, lay.first, 0.0)
        L16 = torch.empty(NC + 1, H, dk, dv, dtype=torch.bfloat16, device=DEV)
        L16[:NC] = B
        L16[NC] = 0
        if use_scan:
            chunked._delta_scan(M, B, alpha, S16, lay, reverse=False)
            chunked._delta_scan(M, B, alpha, L16, lay, reverse=True)
        else:
            state = torch.zeros(lay.n_docs, H, dk, dv, device=DEV)
            for idx, docs in zip(lay.steps, lay.step_docs):
                bgemm(M, S16, b_mn=True, a_index=idx, b_index=idx, out=state, c_index=docs, cin=state, cin_index=docs,
                      gamma=alpha, alpha=-1.0, add16=B, add16_index=idx, out16=S16, out16_index=idx, out16_offset=1,
                      n_hi=len(idx))
            lam = B.index_select(0, lay.last).float()
            for idx, docs in zip(lay.steps[::-1], lay.step_docs[::-1]):
                bgemm(M, L16, a_mn=True, b_mn=True, a_index=idx, b_index=idx, b_offset=1, out=lam, c_index=docs, cin=lam,
                      cin_index=docs, gamma=alpha, alpha=-1.0, add16=B, add16_index=idx, out16=L16, out16_index=idx,
                      n_hi=len(idx))
        outs.append((S16[:NC].float(), L16[:NC].float()))
    from flame_b200.ops import _lib
    _lib.assert_status_ok()
    assert rel_err(outs[0][0], outs[1][0]) < 2e-3
    assert rel_err(outs[0][1], outs[1][1]) < 2e-3


def test_scalar_gla_and_gla_kernels_match_fp32_references():
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.chunked import gla_tc, scalar_gla_tc
    torch.manual_seed(4)
    meta = _meta(LENS)
    T, H, dk, dv = sum(LENS), 2, 128, 128
    leaf = lambda *s: torch.randn(*s, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    q, k, v, graw, gk = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv), leaf(T, H), leaf(T, H, dk)
    ins = [q, k, v, graw]
    ref = _run(lambda c: la.scalar_gla_chunk(c(q), c(k), c(v), -F.softplus(graw.float()) * 0.3, meta, 0.1), ins, True)
    out = _run(lambda c: scalar_gla_tc(c(q), c(k), c(v), -F.softplus(graw.float()) * 0.3, meta, 0.1), ins, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 3e-2
    ins = [q, k, v, gk]
    ref = _run(lambda c: la.gla_chunk(c(q), c(k), c(v), F.logsigmoid(gk.float() * 4), meta), ins, True)
    out = _run(lambda c: gla_tc(c(q), c(k), c(v), F.logsigmoid(gk.float() * 4), meta), ins, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 3e-2


def test_selective_scan_kernels_match_recurrence():
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.scan import selective_scan
    torch.manual_seed(5)
    lens = [70, 1, 64, 130, 17, 300]
    meta = _meta(lens)
    T, Di, N = sum(lens), 96, 16
    u = torch.randn(T, Di, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    draw = torch.randn(T, Di, device=DEV).requires_grad_(True)
    Alog = torch.log(torch.arange(1, N + 1, device=DEV, dtype=torch.float32))[None].repeat(Di, 1).requires_grad_(True)
    B = torch.randn(T, N, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    C = torch.randn(T, N, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    D = torch.randn(Di, device=DEV).requires_grad_(True)
    ins = [u, draw, Alog, B, C, D]

    def run(fn, f32):
        for t in ins:
            t.grad = None
        c = (lambda x: x.float()) if f32 else (lambda x: x)
        y = fn(c(u), F.softplus(draw) * 0.5, -torch.exp(Alog), c(B), c(C), D, meta)
        torch.manual_seed(7)
        (y.float() * torch.randn(y.shape, device=DEV)).sum().backward()
        return [y.detach()] + [t.grad.clone() for t in ins]
    ref = run(la.selective_scan_recurrent, True)
    out = run(selective_scan, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 2e-2


def test_gsa_kernels_match_fp32_chunk_reference():
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.gla import gsa
    torch.manual_seed(6)
    meta = _meta(LENS)
    T, H, dk, M, dv = sum(LENS), 2, 128, 64, 128
    leaf = lambda *s: torch.randn(*s, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    q, k, v, sl, graw = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv), leaf(T, H, M), leaf(T, H, M)
    ins = [q, k, v, sl, graw]
    ref = _run(lambda c: la.gsa_chunk(c(q), c(k), c(v), c(sl), F.logsigmoid(graw.float()) / 8, meta), ins, True)
    out = _run(lambda c: gsa(c(q), c(k), c(v), c(sl), F.logsigmoid(graw.float()) / 8, meta), ins, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 4e-2


def test_mamba2_ssd_grouped_heads_match_recurrence():
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.scan import mamba2_ssd
    torch.manual_seed(8)
    lens = [70, 1, 64, 130, 17, 200]
    meta = _meta(lens)
    T, H, P, N, G = sum(lens), 8, 64, 128, 2
    leaf = lambda *s: torch.randn(*s, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    x, dtraw, B, C = leaf(T, H, P), leaf(T, H), leaf(T, G, N), leaf(T, G, N)
    A = -torch.rand(H, device=DEV) * 2 - 0.5
    D = torch.randn(H, device=DEV)
    ins = [x, dtraw, B, C]
    ref = _run(lambda c: la.mamba2_ssd_recurrent(c(x), F.softplus(dtraw.float()) * 0.3, A, c(B) * 0.2, c(C) * 0.2, D, meta), ins, True)
    out = _run(lambda c: mamba2_ssd(c(x), F.softplus(dtraw.float()) * 0.3, A, c(B) * 0.2, c(C) * 0.2, D, meta), ins, False)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 3e-2
