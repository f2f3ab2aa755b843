"""Float8 linear layers without a GPU: the torch-float8 path of ``ops/float8.py`` against fp32 matmuls.

Counterpart of the reference's float8 converter (torchtitan/components/quantization/float8.py), whose arithmetic
(tensor-wise dynamic scales, e4m3 activations / weights, e5m2 output gradients) these tests pin down.
"""
import pytest
import torch

from flame_b200.ops import float8
from flame_b200.ops.linear import linear, linear_fused


def test_quantize_roundtrip_and_transpose():
    torch.manual_seed(0)
    x = (torch.randn(64, 48) * 3).to(torch.bfloat16)
    for dtype, tol in ((float8.E4M3, 2 ** -4), (float8.E5M2, 2 ** -3)):
        q, qT, inv = float8.quantize(x, dtype)
        assert q.dtype == dtype and q.shape == (64, 48) and qT.shape == (48, 64)
        assert torch.equal(qT.float(), q.float().t())
        back = q.float() * inv
        # relative spacing of the format bounds the error of every element that is not tiny
        big = x.float().abs() > x.float().abs().max() / 64
        rel = ((back - x.float()).abs() / x.float().abs())[big].max()
        assert rel <= tol, (dtype, rel)
        # the largest element maps to the format's largest finite value
        assert torch.isclose(q.float().abs().max(), torch.tensor(float8._FMAX[dtype]))


def test_gemm_fp8_matches_dequantised_matmul():
    torch.manual_seed(1)
    a = torch.randn(32, 64).to(torch.bfloat16)
    b = torch.randn(48, 64).to(torch.bfloat16)
    aq, _, ai = float8.quantize(a)
    bq, _, bi = float8.quantize(b, float8.E5M2)
    out = float8.gemm_fp8(aq, bq, ai, bi, out_dtype=torch.float32)
    ref = (aq.float() * ai) @ (bq.float() * bi).t()
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    acc = torch.ones(32, 48)
    float8.gemm_fp8(aq, bq, ai, bi, out=acc, accumulate=True)
    torch.testing.assert_close(acc, ref + 1, rtol=1e-5, atol=1e-5)


def test_float8_linear_forward_backward_close_to_fp32():
    torch.manual_seed(2)
    x = torch.randn(4, 16, 64, dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(96, 64, dtype=torch.bfloat16) * 0.1)
    w._fp8 = True
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    assert rel(y, yr) < 0.05
    assert rel(x.grad, xr.grad) < 0.08
    assert rel(w.grad, wr.grad) < 0.08


def test_float8_fused_projections_and_main_grad():
    torch.manual_seed(3)
    x = torch.randn(32, 64, dtype=torch.bfloat16, requires_grad=True)
    ws = [torch.nn.Parameter(torch.randn(32, 64, dtype=torch.bfloat16) * 0.1) for _ in range(3)]
    for w in ws:
        w._fp8 = True
        w.main_grad = torch.zeros(32, 64)
    y = linear_fused(x, ws)
    assert y.shape == (32, 96)
    y.float().sum().backward()
    ref = torch.cat([x.detach().float() @ w.detach().float().t() for w in ws], -1)
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.05
    for w in ws:
        assert w.grad is None  # the engine's contract: the gradient went into main_grad
        wref = torch.ones(32, 32) .t() @ x.detach().float()
        assert ((w.main_grad - wref).norm() / wref.norm()).item() < 0.08


def test_converter_marks_projections_only():
    from flame_b200.models import ModelConfig, build_model
    cfg = ModelConfig.from_dict(dict(model_type="transformer", hidden_size=64, num_hidden_layers=2, num_heads=4,
                                     vocab_size=128, intermediate_size=128))
    model = build_model(cfg, device="cpu", dtype=torch.float32)
    n = float8.convert_to_float8(model)
    marked = [name for name, p in model.named_parameters() if getattr(p, "_fp8", False)]
    assert n == len(marked) > 0
    assert all("lm_head" not in m and "embed" not in m and "norm" not in m for m in marked)
    assert any("q_proj" in m for m in marked) and any("down_proj" in m for m in marked)


@pytest.mark.parametrize("recipe", ["rowwise", "rowwise_with_gw_hp"])
def test_rowwise_recipes_forward_backward_close_to_fp32(recipe):
    """One power-of-two scale per row of every operand (the reference converter's row-wise recipes)."""
    torch.manual_seed(4)
    x = torch.randn(64, 64, dtype=torch.bfloat16)
    x[3] *= 50.0    # an outlier token: a tensor-wise scale would crush every other row, a per-row scale does not
    x.requires_grad_(True)
    w = torch.nn.Parameter(torch.randn(96, 64, dtype=torch.bfloat16) * 0.1)
    w._fp8 = recipe
    w.main_grad = torch.zeros(96, 64)
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(g.float())

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    rows = [i for i in range(64) if i != 3]
    assert rel(y[rows], (xr @ wr.t()).detach()[rows]) < 0.05          # the ordinary rows keep their precision
    assert rel(x.grad, xr.grad) < 0.08
    assert rel(w.main_grad, wr.grad) < (0.02 if recipe == "rowwise_with_gw_hp" else 0.08)
    q, inv = float8.quantize_rows(x.detach())
    assert torch.equal(torch.log2(inv), torch.log2(inv).round())      # power-of-two scales
    assert float(q.float().abs().max()) <= float8._FMAX[float8.E4M3]


def test_converter_takes_the_recipe_names():
    from flame_b200.models import ModelConfig, build_model
    cfg = ModelConfig.from_dict(dict(model_type="transformer", hidden_size=64, num_hidden_layers=1, num_heads=4,
                                     vocab_size=128, intermediate_size=128))
    model = build_model(cfg, device="cpu", dtype=torch.float32)
    assert float8.convert_to_float8(model, recipe="rowwise") > 0
    assert {getattr(p, "_fp8", None) for n, p in model.named_parameters() if "q_proj" in n} == {"rowwise"}
    with pytest.raises(ValueError):
        float8.convert_to_float8(model, recipe="columnwise")
