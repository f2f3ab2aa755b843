"""fp8 quantisation kernels and the kind::f8f6f4 GEMM against fp32 PyTorch on the same values."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cuda():
    from flame_b200.ops import _lib
    assert torch.cuda.is_available() and _lib.available(), "the fp8 tests need the built library on a GPU"


@pytest.mark.parametrize("rows,cols", [(256, 128), (1040, 336), (4096, 1024)])
@pytest.mark.parametrize("e5m2", [False, True])
def test_quantize_kernel(rows, cols, e5m2):
    _cuda()
    from flame_b200.ops import float8
    torch.manual_seed(rows + cols)
    dtype = float8.E5M2 if e5m2 else float8.E4M3
    x = (torch.randn(rows, cols, device="cuda") * 2.5).to(torch.bfloat16)
    q, qT, inv = float8.quantize(x, dtype)
    fmax = float8._FMAX[dtype]
    amax = x.float().abs().max()
    torch.testing.assert_close(inv, (amax / fmax).reshape(1), rtol=1e-6, atol=0)
    # Correct rounding, whichever way ties go (x values that are simple fractions of amax land exactly between two
    # fp8 values, and a one-ulp difference in the scale decides those): every element is within half a spacing of
    # the scaled fp32 value, and almost all agree with torch's own cast.
    v = (x.float() * (fmax / amax)).clamp(-fmax, fmax)
    mant, emin = (2, -14) if e5m2 else (3, -6)
    expo = torch.floor(torch.log2(v.abs().clamp_min(2.0 ** emin))).clamp_min(emin)
    spacing = torch.exp2(expo - mant)
    assert ((q.float() - v).abs() <= 0.5 * spacing * (1 + 1e-3)).all()
    mism = (q.float() != v.to(dtype).float()).float().mean().item()
    assert mism < 0.03, mism
    assert torch.equal(qT.view(torch.uint8), q.view(torch.uint8).t().contiguous())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1024, 768, 1040), (4096, 1024, 4096), (272, 48, 4096)])
@pytest.mark.parametrize("b_e5m2", [False, True])
def test_gemm_fp8(M, N, K, b_e5m2):
    _cuda()
    from flame_b200.ops import _lib, float8
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    aq, _, ai = float8.quantize(a, float8.E4M3, transpose=False)
    bq, _, bi = float8.quantize(b, float8.E5M2 if b_e5m2 else float8.E4M3, transpose=False)
    ref = (aq.float() * ai) @ (bq.float() * bi).t()
    out = float8.gemm_fp8(aq, bq, ai, bi, out_dtype=torch.float32)
    _lib.assert_status_ok()
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-3 * ref.abs().max().item())
    out16 = float8.gemm_fp8(aq, bq, ai, bi)
    torch.testing.assert_close(out16.float(), ref, rtol=2e-2, atol=1e-2 * ref.abs().max().item())
    acc = torch.full((M, N), 0.5, device="cuda")
    float8.gemm_fp8(aq, bq, ai, bi, out=acc, accumulate=True)
    torch.testing.assert_close(acc, ref + 0.5, rtol=2e-3, atol=2e-3 * ref.abs().max().item())
    _lib.assert_status_ok()


def test_float8_linear_matches_bf16_linear():
    _cuda()
    from flame_b200.ops.linear import linear
    torch.manual_seed(7)
    x = torch.randn(2048, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w8 = torch.nn.Parameter(torch.randn(3072, 1024, device="cuda", dtype=torch.bfloat16) * 0.03)
    w8._fp8 = True
    w8.main_grad = torch.zeros(3072, 1024, device="cuda")
    g = torch.randn(2048, 3072, device="cuda", dtype=torch.bfloat16)
    y8 = linear(x, w8)
    y8.backward(g)
    dx8 = x.grad.clone()
    xr = x.detach().float().requires_grad_()
    wr = w8.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    assert rel(y8, yr) < 0.05
    assert rel(dx8, xr.grad) < 0.08
    assert w8.grad is None
    assert rel(w8.main_grad, wr.grad) < 0.08


def test_float8_training_step_through_engine():
    """A converted model takes optimizer steps through the engine and its loss falls on a fixed batch."""
    _cuda()
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.ops.float8 import convert_to_float8
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    torch.manual_seed(0)
    cfg = ModelConfig("transformer", hidden_size=256, num_hidden_layers=2, vocab_size=512,
                      max_position_embeddings=4096, num_heads=4)
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    assert convert_to_float8(model) > 0
    eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device("cuda"), torch.bfloat16,
                        OptimConfig(lr=3e-3, weight_decay=0.0, max_norm=1.0, skip_nan_inf=True))
    eng.init_weights(0)
    model.train()
    assert any(getattr(p, "_fp8", False) for p in model.parameters())
    lens = [304, 80, 128, 512]  # fp8 operands need a token count that is a multiple of 16
    ids = torch.randint(3, 512, (1, sum(lens)), device="cuda")
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    _lib.status_clear()
    losses = []
    for _ in range(30):
        eng.zero_grad()
        out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
        out.loss.backward()
        eng.step(3e-3)
        losses.append(float(out.loss.detach()))
    torch.cuda.synchronize()
    assert _lib.status() == 0
    assert eng.skipped_steps() == 0
    assert losses[-1] < losses[0] - 1.5, (losses[0], losses[-1])


@pytest.mark.parametrize("recipe", ["rowwise", "rowwise_with_gw_hp"])
def test_rowwise_recipes_on_the_fp8_gemm(recipe):
    """One power-of-two scale per operand row, applied to the fp8 GEMM's fp32 result: close to the bf16 layer, and an
    outlier token does not cost the other rows their precision."""
    _cuda()
    from flame_b200.ops.linear import linear
    torch.manual_seed(11)
    T, K, N = 1024, 512, 768
    x = torch.randn(T, K, device="cuda").bfloat16()
    x[5] *= 60.0
    x.requires_grad_(True)
    w = torch.nn.Parameter((torch.randn(N, K, device="cuda") * 0.05).bfloat16())
    w._fp8 = recipe
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    rows = [i for i in range(T) if i != 5]
    assert rel(y[rows], yr.detach()[rows]) < 0.05
    assert rel(x.grad, xr.grad) < 0.08
    assert rel(w.grad, wr.grad) < (0.02 if recipe == "rowwise_with_gw_hp" else 0.08)
