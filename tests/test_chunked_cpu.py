"""The batched-GEMM chunk algorithms (gated delta rule, scalar-gated and per-channel-gated linear attention) against
their token-by-token definitions, forward and backward, on the CPU reference path of ``ops.bgemm`` (fp32)."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err
from flame_b200.ops import linear_attn as la
from flame_b200.ops.bgemm import MASK_TRIL, bgemm, bmm
from flame_b200.ops.chunked import ChunkLayout, gated_delta_rule_tc, gla_tc, scalar_gla_tc
from flame_b200.ops.varlen import VarlenMeta


def _meta(lens):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return VarlenMeta.from_cu_seqlens(cu, sum(lens))


LENS = [70, 1, 64, 130, 17]


def _leaf(*shape):
    return torch.randn(*shape).requires_grad_(True)


def _run(fn, inputs):
    for t in inputs:
        t.grad = None
    o = fn()
    torch.manual_seed(99)
    (o * torch.randn_like(o)).sum().backward()
    return [o.detach()] + [t.grad.clone() for t in inputs]


def test_chunk_layout_pack_unpack_roundtrip():
    meta = _meta(LENS)
    lay = ChunkLayout.of(meta)
    assert lay.NC == sum((n + 63) // 64 for n in LENS)
    x = torch.randn(sum(LENS), 3, 5)
    p = lay.pack(x)
    assert p.shape == (lay.NC, 64, 3, 5)
    assert torch.equal(lay.unpack(p), x)
    assert p.abs().sum().item() == pytest.approx(x.abs().sum().item(), rel=1e-5)  # padding rows are zero
    # chunk positions: every listed chunk has its successor in the same document
    first = set(lay.first.tolist())
    for s, idx in enumerate(lay.steps):
        for c in idx.tolist():
            assert (c + 1) not in first


def test_bgemm_reference_layouts_and_bmm_gradients():
    torch.manual_seed(0)
    a = torch.randn(3, 2, 8, 5, requires_grad=True)       # [hi, lo, M, K]
    bt = torch.randn(3, 2, 5, 7, requires_grad=True)      # [hi, lo, K, N]  (mn storage)
    out = bmm(a, bt, b_mn=True, alpha=0.5)
    ref = 0.5 * a @ bt
    assert rel_err(out, ref) < 1e-6
    g = torch.randn_like(out)
    ga, gb = torch.autograd.grad(out, (a, bt), g)
    ra, rb = torch.autograd.grad(ref, (a, bt), g)
    assert rel_err(ga, ra) < 1e-6 and rel_err(gb, rb) < 1e-6
    # masked, decayed scores
    q, k = torch.randn(2, 2, 6, 4), torch.randn(2, 2, 6, 4)
    d = -torch.rand(2, 2, 6).cumsum(-1)
    s = bgemm(q, k, decay=d, mask=MASK_TRIL)
    full = (q @ k.transpose(-1, -2)) * (d[..., :, None] - d[..., None, :]).exp()
    assert rel_err(s, full.tril()) < 1e-6


@pytest.mark.parametrize("gated,chunk", [(True, 128), (False, 128), (True, 64)])
def test_gated_delta_rule_tc_matches_recurrence(gated, chunk):
    torch.manual_seed(2)
    meta = _meta(LENS)
    T, H, K, V = sum(LENS), 2, 16, 24
    q, k, v, braw, graw = _leaf(T, H, K), _leaf(T, H, K), _leaf(T, H, V), _leaf(T, H), _leaf(T, H)
    ins = [q, k, v, braw] + ([graw] if gated else [])

    def make(fn):
        def f():
            g = -F.softplus(graw) if gated else None
            return fn(la.l2norm(q), la.l2norm(k), v, braw.sigmoid(), g, meta)
        return f
    ref = _run(make(la.gated_delta_rule_recurrent), ins)
    out = _run(make(lambda *a: gated_delta_rule_tc(*a, chunk=chunk)), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4


def test_scalar_gla_tc_matches_chunk_reference():
    torch.manual_seed(3)
    meta = _meta(LENS)
    T, H, K, V = sum(LENS), 3, 16, 8
    q, k, v, graw = _leaf(T, H, K), _leaf(T, H, K), _leaf(T, H, V), _leaf(T, H)
    ins = [q, k, v, graw]
    ref = _run(lambda: la.scalar_gla_chunk(q, k, v, -F.softplus(graw), meta, 0.3), ins)
    out = _run(lambda: scalar_gla_tc(q, k, v, -F.softplus(graw), meta, 0.3), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4


def test_gla_tc_matches_recurrence_with_strong_gates():
    torch.manual_seed(4)
    meta = _meta(LENS)
    T, H, K, V = sum(LENS), 2, 16, 24
    q, k, v, graw = _leaf(T, H, K), _leaf(T, H, K), _leaf(T, H, V), _leaf(T, H, K)
    ins = [q, k, v, graw]
    ref = _run(lambda: la.gla_recurrent(q, k, v, F.logsigmoid(graw * 8), meta), ins)   # decays down to e^-20 per step
    out = _run(lambda: gla_tc(q, k, v, F.logsigmoid(graw * 8), meta), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4
    assert all(torch.isfinite(t).all() for t in out)


def test_gla_vdecay_tc_and_gsa_match_recurrence():
    from flame_b200.ops.chunked import gla_vdecay_tc
    from flame_b200.ops.gla import gsa
    torch.manual_seed(5)
    meta = _meta(LENS)
    T, H, K, M = sum(LENS), 2, 16, 8
    q, k, s, graw = _leaf(T, H, K), _leaf(T, H, K), _leaf(T, H, M), _leaf(T, H, M)
    ins = [q, k, s, graw]
    ref = _run(lambda: la.gla_recurrent_vdecay(q, k, s, F.logsigmoid(graw * 4), meta, 0.25), ins)
    out = _run(lambda: gla_vdecay_tc(q, k, s, F.logsigmoid(graw * 4), meta, 0.25), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4
    v = _leaf(T, H, 12)
    ins = [q, k, v, s, graw]
    ref = _run(lambda: la.gsa_recurrent(q, k, v, s, F.logsigmoid(graw) / 8, meta), ins)
    out = _run(lambda: gsa(q, k, v, s, F.logsigmoid(graw) / 8, meta), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4


def test_mamba2_ssd_grouped_matches_recurrence():
    from flame_b200.ops.scan import mamba2_ssd
    torch.manual_seed(6)
    meta = _meta(LENS)
    T, H, P, N, G = sum(LENS), 4, 8, 16, 2
    x, dtraw, B, C = _leaf(T, H, P), _leaf(T, H), _leaf(T, G, N), _leaf(T, G, N)
    A = -torch.rand(H) * 2 - 0.5
    D = torch.randn(H)
    ins = [x, dtraw, B, C]
    ref = _run(lambda: la.mamba2_ssd_recurrent(x, F.softplus(dtraw), A, B, C, D, meta), ins)
    out = _run(lambda: mamba2_ssd(x, F.softplus(dtraw), A, B, C, D, meta), ins)
    for a, b in zip(out, ref):
        assert rel_err(a, b) < 1e-4


def test_chunk_layout_arrays_match_a_per_token_construction():
    """The array-built layout (rows, inverse map, first / last chunks, per-position lists) against the obvious loops."""
    from flame_b200.ops.chunked import ChunkLayout
    lens = [1, 63, 64, 65, 130, 7]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    meta = VarlenMeta.from_cu_seqlens(cu, sum(lens), torch.device("cpu"))
    lay = ChunkLayout(meta, 64)
    rows, first, last, c0 = [], [], [], 0
    steps = {}
    for d, n in enumerate(lens):
        nc = (n + 63) // 64
        rows += list(range(c0 * 64, c0 * 64 + n))
        first.append(c0)
        last.append(c0 + nc - 1)
        for s_ in range(nc - 1):
            steps.setdefault(s_, []).append((c0 + s_, d))
        c0 += nc
    assert lay.NC == c0 and lay.T == sum(lens) and lay.Tp == c0 * 64 and not lay.aligned
    assert lay.rows.tolist() == rows and lay.first.tolist() == first and lay.last.tolist() == last
    inv = [-1] * (c0 * 64)
    for t_, r in enumerate(rows):
        inv[r] = t_
    assert lay.inv_i32.tolist() == inv
    assert [s.tolist() for s in lay.steps] == [[c for c, _ in steps[k]] for k in sorted(steps)]
    assert [d.tolist() for d in lay.step_docs] == [[d for _, d in steps[k]] for k in sorted(steps)]
    x = torch.randn(sum(lens), 3, requires_grad=True)
    packed = lay.pack(x)
    assert packed.shape == (c0, 64, 3)
    assert torch.equal(lay.unpack(packed), x)
    assert float(packed.detach().reshape(-1, 3)[[i for i, v in enumerate(inv) if v < 0]].abs().sum()) == 0.0
    packed.square().sum().backward()
    assert torch.allclose(x.grad, 2 * x.detach())


def test_column_split_writes_one_gradient_matrix():
    from flame_b200.ops.gates import split_columns
    x = torch.randn(5, 9, requires_grad=True)
    a, b, c = split_columns(x, (2, 4, 3))
    (a.sum() * 2 + (c * c).sum()).backward()      # the middle block gets no gradient at all
    ref = torch.zeros(5, 9)
    ref[:, :2] = 2
    ref[:, 6:] = 2 * x.detach()[:, 6:]
    assert torch.equal(x.grad, ref)
