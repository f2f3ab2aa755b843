"""Chunk-parallel PyTorch token mixers against their token-by-token definitions (CPU, fp32)."""
import torch

from conftest import rel_err
from flame_b200.ops import linear_attn as la
from flame_b200.ops.varlen import VarlenMeta


def _meta(lens):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return VarlenMeta.from_cu_seqlens(cu, sum(lens))


LENS = [70, 1, 64, 130, 17]


def test_gla_chunk_matches_recurrence():
    torch.manual_seed(0)
    meta = _meta(LENS)
    T, H, K, V = sum(LENS), 2, 16, 24
    q, k, v = torch.randn(T, H, K), torch.randn(T, H, K), torch.randn(T, H, V)
    g = torch.nn.functional.logsigmoid(torch.randn(T, H, K) * 3)  # includes strong decays
    ref = la.gla_recurrent(q, k, v, g, meta)
    out = la.gla_chunk(q, k, v, g, meta)
    assert rel_err(out, ref) < 1e-4


def test_scalar_gla_and_mamba2():
    torch.manual_seed(1)
    meta = _meta(LENS)
    T, H, P, N = sum(LENS), 4, 8, 16
    x = torch.randn(T, H, P)
    dt = torch.nn.functional.softplus(torch.randn(T, H))
    A = -torch.rand(H) * 4 - 0.5
    B, C = torch.randn(T, 1, N), torch.randn(T, 1, N)
    D = torch.randn(H)
    ref = la.mamba2_ssd_recurrent(x, dt, A, B, C, D, meta)
    out = la.mamba2_ssd(x, dt, A, B, C, D, meta)
    assert rel_err(out, ref) < 1e-4


def test_gated_delta_rule_chunk_matches_recurrence():
    torch.manual_seed(2)
    meta = _meta(LENS)
    T, H, K, V = sum(LENS), 2, 16, 32
    q, k = la.l2norm(torch.randn(T, H, K)), la.l2norm(torch.randn(T, H, K))
    v = torch.randn(T, H, V)
    beta = torch.sigmoid(torch.randn(T, H))
    g = -torch.rand(T, H) * 0.5
    ref = la.gated_delta_rule_recurrent(q, k, v, beta, g, meta)
    out = la.gated_delta_rule_chunk(q, k, v, beta, g, meta)
    assert rel_err(out, ref) < 1e-4
    ref0 = la.gated_delta_rule_recurrent(q, k, v, beta, None, meta)
    out0 = la.gated_delta_rule_chunk(q, k, v, beta, None, meta)
    assert rel_err(out0, ref0) < 1e-4


def test_gsa_chunk_matches_recurrence():
    torch.manual_seed(3)
    meta = _meta(LENS)
    T, H, K, V, M = sum(LENS), 2, 16, 16, 8
    q, k, v = torch.randn(T, H, K), torch.randn(T, H, K), torch.randn(T, H, V)
    f = torch.nn.functional.logsigmoid(torch.randn(T, H, M)) / 4
    s = 1 - f.exp()
    ref = la.gsa_recurrent(q, k, v, s, f, meta)
    out = la.gsa_chunk(q, k, v, s, f, meta)
    assert rel_err(out, ref) < 1e-4


def test_selective_scan_chunk_matches_recurrence():
    torch.manual_seed(4)
    meta = _meta([70, 3, 64])
    T, Di, N = 137, 12, 4
    u = torch.randn(T, Di)
    delta = torch.nn.functional.softplus(torch.randn(T, Di))
    A = -torch.rand(Di, N) * 3 - 0.1
    B, C = torch.randn(T, N), torch.randn(T, N)
    D = torch.randn(Di)
    ref = la.selective_scan_recurrent(u, delta, A, B, C, D, meta)
    out = la.selective_scan(u, delta, A, B, C, D, meta)
    assert rel_err(out, ref) < 1e-4


def test_short_conv_respects_boundaries():
    torch.manual_seed(5)
    meta = _meta([5, 9, 2])
    T, D, W = 16, 6, 4
    x = torch.randn(T, D)
    w = torch.randn(D, 1, W)
    b = torch.randn(D)
    out = la.short_conv(x, w, b, meta, activation=None)
    ref = torch.zeros_like(out)
    for a, e in [(0, 5), (5, 14), (14, 16)]:
        seg = x[a:e].t()[None]
        y = torch.nn.functional.conv1d(torch.nn.functional.pad(seg, (W - 1, 0)), w, b, groups=D)
        ref[a:e] = y[0].t()
    assert rel_err(out, ref) < 1e-5


def test_stickbreaking_rows_sum_to_at_most_one():
    torch.manual_seed(6)
    meta = _meta([33, 8])
    q, k, v = torch.randn(41, 2, 16), torch.randn(41, 2, 16), torch.randn(41, 2, 16)
    o, rem = la.stickbreaking_reference(q, k, v, meta)
    assert o.shape == (41, 2, 16)
    assert (rem >= -1e-5).all() and (rem <= 1 + 1e-5).all()
    assert torch.allclose(rem[0], torch.ones(2)) and torch.allclose(rem[33], torch.ones(2))


# ---------------------------------------------------------------------------------------------------------------
# the same recurrences as written by the reference's kernel library (fla.ops.*.naive, pure PyTorch, CPU)
# ---------------------------------------------------------------------------------------------------------------
def _fla_naive(path):
    import importlib
    import pytest
    try:
        return importlib.import_module(path)
    except Exception as e:
        pytest.skip(f"{path} is not importable: {e!r}")


def _bt(x):  # packed [T, ...] single document -> the reference's [B = 1, T, ...]
    return x.unsqueeze(0)


def test_oracles_agree_with_the_reference_library_recurrences():
    torch.manual_seed(11)
    T, H, K, V, M = 96, 2, 16, 24, 8
    meta = _meta([T])
    q, k, v = torch.randn(T, H, K), la.l2norm(torch.randn(T, H, K)), torch.randn(T, H, V)
    beta = torch.rand(T, H)
    g = torch.nn.functional.logsigmoid(torch.randn(T, H) * 2)
    # gated delta rule (fla/ops/gated_delta_rule/naive.py:13-64) and the plain delta rule (fla/ops/delta_rule/naive.py:12-37)
    m = _fla_naive("fla.ops.gated_delta_rule.naive")
    ref, _ = m.naive_recurrent_gated_delta_rule(_bt(q), _bt(k), _bt(v), _bt(beta), _bt(g))
    assert rel_err(la.gated_delta_rule_recurrent(q, k, v, beta, g, meta), ref[0]) < 1e-5
    assert rel_err(la.gated_delta_rule_chunk(q, k, v, beta, g, meta), ref[0]) < 1e-4
    m = _fla_naive("fla.ops.delta_rule.naive")
    ref, _ = m.delta_rule_recurrence(_bt(q).transpose(1, 2), _bt(k).transpose(1, 2), _bt(v).transpose(1, 2),
                                     _bt(beta).transpose(1, 2))
    assert rel_err(la.gated_delta_rule_recurrent(q, k, v, beta, None, meta), ref[0].transpose(0, 1)) < 1e-5
    # GLA (fla/ops/gla/naive.py:15-45)
    gk = torch.nn.functional.logsigmoid(torch.randn(T, H, K) * 2)
    m = _fla_naive("fla.ops.gla.naive")
    ref, _ = m.naive_recurrent_gla(_bt(q), _bt(k), _bt(v), _bt(gk))
    assert rel_err(la.gla_recurrent(q, k, v, gk, meta), ref[0]) < 1e-5
    assert rel_err(la.gla_chunk(q, k, v, gk, meta), ref[0]) < 1e-4
    # GSA (fla/ops/gsa/naive.py:12-70)
    s = torch.randn(T, H, M)
    gs = torch.nn.functional.logsigmoid(torch.randn(T, H, M))
    m = _fla_naive("fla.ops.gsa.naive")
    ref = m.naive_recurrent_gsa(_bt(q), _bt(k), _bt(v), _bt(s), _bt(gs))
    ref = ref[0] if isinstance(ref, tuple) else ref
    assert rel_err(la.gsa_recurrent(q, k, v, s, gs, meta), ref[0]) < 1e-5
    assert rel_err(la.gsa_chunk(q, k, v, s, gs, meta), ref[0]) < 1e-4


def test_stickbreaking_oracle_agrees_with_the_reference_formula():
    """custom_models/sba/stickbreaking_attention/sb_ref.py:8-25, loaded from the installed (unmodified) reference."""
    import importlib.util
    import os
    import pytest
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "custom_models",
                        "sba", "stickbreaking_attention", "sb_ref.py")
    if not os.path.isfile(path):
        pytest.skip("the reference's custom model is not installed under baseline/_ref")
    spec = importlib.util.spec_from_file_location("sb_ref", path)
    sb_ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sb_ref)
    torch.manual_seed(12)
    T, H, D = 80, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, H, D), torch.randn(T, H, D)
    mask = torch.ones(T, T).triu(0).bool()            # a key at or after the query is masked
    cum_weight = torch.ones(T, T).tril(-1)            # sum over the keys strictly after j
    ref_o, ref_rem = sb_ref.stickbreaking(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                          mask[None, None], cum_weight)
    o, rem = la.stickbreaking_reference(q, k, v, _meta([T]))
    assert rel_err(o, ref_o[0].transpose(0, 1)) < 1e-5
    assert (rem - ref_rem[0].transpose(0, 1)).abs().max() < 1e-5
