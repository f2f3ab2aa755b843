"""Edge-length documents and run-to-run repeatability of the CUDA kernels (``pytest -m gpu``).

Document lengths straddle every tile size used by the kernels (16-row sub-blocks, 64 / 128-token chunks and
attention tiles); kernels whose reductions have a fixed order must reproduce their output bit for bit, which doubles
as a race detector on a pool where compute-sanitizer is not available."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
EDGE_LENS = [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 2, 255, 256, 257]


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


def _leaf(*s):
    return torch.randn(*s, device=DEV, dtype=torch.bfloat16).requires_grad_(True)


def test_attention_edge_lengths():
    from flame_b200.ops.attention import attention, attention_reference
    torch.manual_seed(0)
    meta = _meta(EDGE_LENS)
    T, H, D = sum(EDGE_LENS), 2, 64
    q, k, v = _leaf(T, H, D), _leaf(T, H, D), _leaf(T, H, D)
    o = attention(q, k, v, meta)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    oref = attention_reference(qf, kf, vf, meta, D ** -0.5)
    assert rel_err(o, oref) < 1e-2
    do = torch.randn_like(o)
    o.backward(do)
    oref.backward(do.float())
    for a, b in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert rel_err(a, b) < 2e-2


def test_chunk_algorithms_edge_lengths():
    from flame_b200.ops import linear_attn as la
    from flame_b200.ops.chunked import gated_delta_rule_tc, gla_tc
    torch.manual_seed(1)
    meta = _meta(EDGE_LENS)
    T, H, dk, dv = sum(EDGE_LENS), 2, 128, 128
    q, k, v, braw, graw, gk = _leaf(T, H, dk), _leaf(T, H, dk), _leaf(T, H, dv), _leaf(T, H), _leaf(T, H), _leaf(T, H, dk)
    g = -F.softplus(graw.float()) * 0.3
    beta = braw.float().sigmoid()
    for chunk in (64, 128):
        o = gated_delta_rule_tc(la.l2norm(q), la.l2norm(k), v, beta, g, meta, chunk=chunk)
        ref = la.gated_delta_rule_chunk(la.l2norm(q.float()), la.l2norm(k.float()), v.float(), beta, g, meta)
        assert torch.isfinite(o).all() and rel_err(o, ref) < 2e-2
    o = gla_tc(q, k, v, F.logsigmoid(gk.float() * 4), meta)
    ref = la.gla_chunk(q.float(), k.float(), v.float(), F.logsigmoid(gk.float() * 4), meta)
    assert torch.isfinite(o).all() and rel_err(o, ref) < 2e-2


def test_fixed_order_kernels_repeat_bitwise():
    from flame_b200.ops import gemm
    from flame_b200.ops.attention import attention
    from flame_b200.ops.bgemm import MASK_TRIL, bgemm
    from flame_b200.ops.chunked import gated_delta_rule_tc
    from flame_b200.ops.norm import rms_norm
    torch.manual_seed(2)
    a, b = torch.randn(1000, 520, device=DEV).bfloat16(), torch.randn(776, 520, device=DEV).bfloat16()
    assert torch.equal(gemm.gemm_nt(a, b), gemm.gemm_nt(a, b))
    dy, x = torch.randn(8192, 256, device=DEV).bfloat16(), torch.randn(8192, 512, device=DEV).bfloat16()
    assert torch.equal(gemm.gemm_tn(dy, x, out_dtype=torch.float32), gemm.gemm_tn(dy, x, out_dtype=torch.float32))  # split-K
    meta = _meta([300, 77, 129, 1, 1000])
    T = meta.total_tokens
    q, k, v = (torch.randn(T, 2, 64, device=DEV).bfloat16() for _ in range(3))
    assert torch.equal(attention(q, k, v, meta), attention(q, k, v, meta))
    qq = torch.randn(9, 64, 3, 128, device=DEV).bfloat16().permute(0, 2, 1, 3)
    d = (-torch.rand(9, 64, 3, device=DEV)).cumsum(1).permute(0, 2, 1)
    assert torch.equal(bgemm(qq, qq, decay=d, mask=MASK_TRIL), bgemm(qq, qq, decay=d, mask=MASK_TRIL))
    # RMSNorm weight gradient: per-CTA partials summed in a fixed order
    xn = torch.randn(5000, 1024, device=DEV).bfloat16().requires_grad_(True)
    w = torch.ones(1024, device=DEV).bfloat16().requires_grad_(True)
    gsum = []
    for _ in range(2):
        xn.grad = w.grad = None
        rms_norm(xn, w, 1e-6).backward(torch.ones(5000, 1024, device=DEV).bfloat16() * 0.5)
        gsum.append((xn.grad.clone(), w.grad.clone()))
    assert torch.equal(gsum[0][0], gsum[1][0]) and torch.equal(gsum[0][1], gsum[1][1])
    # a whole chunk algorithm (batched GEMMs, triangular inverse, state recurrence), forward and backward
    q2, k2, v2 = _leaf(T, 2, 128), _leaf(T, 2, 128), _leaf(T, 2, 128)
    beta = torch.rand(T, 2, device=DEV)
    g = -torch.rand(T, 2, device=DEV) * 0.1
    outs = []
    for _ in range(2):
        q2.grad = k2.grad = v2.grad = None
        o = gated_delta_rule_tc(F.normalize(q2.float(), dim=-1).bfloat16(), F.normalize(k2.float(), dim=-1).bfloat16(), v2,
                                beta, g, meta)
        o.sum().backward()
        outs.append((o.detach().clone(), v2.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_kernels_leave_the_memory_around_their_outputs_alone():
    """Canaries: outputs are views into a larger buffer filled with a sentinel; after the kernels ran, everything outside
    the view still holds the sentinel (tile sizes never divide these shapes, so every kernel has partial tiles)."""
    from flame_b200.ops import gemm
    from flame_b200.ops.attn_block import qkv_attention
    torch.manual_seed(1)
    SENT = -12345.0

    def guarded(rows, cols, dtype):
        big = torch.full((rows + 64, cols), SENT, device=DEV, dtype=dtype)
        return big, big[32:32 + rows]

    def intact(big, rows):
        return bool((big[:32] == SENT).all()) and bool((big[32 + rows:] == SENT).all())

    # GEMMs with out= (bf16 store, fp32 store, fp32 accumulate) at shapes that leave partial tiles in M and N
    M, N, K = 1000, 328, 264
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    for dtype, acc in ((torch.bfloat16, False), (torch.float32, False), (torch.float32, True)):
        big, out = guarded(M, N, dtype)
        if acc:
            out.zero_()
        gemm.gemm_nt(a, b, out=out, accumulate=acc)
        torch.cuda.synchronize()
        assert intact(big, M), (dtype, acc)
        assert rel_err(out.float(), a.float() @ b.float().t()) < 1e-2
    # weight-gradient form (A and B read MN-major), output N x K
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    big, out = guarded(N, K, torch.float32)
    gemm.gemm_tn(dy, a, out=out)
    torch.cuda.synchronize()
    assert intact(big, N)
    assert rel_err(out, dy.float().t() @ a.float()) < 1e-2
    # attention reading q, k, v as strided views of a guarded fused buffer (RoPE rotates q and k in place)
    lens = [1, 127, 129, 300, 65]
    T, H, Dh = sum(lens), 4, 64
    big, qkv = guarded(T, 3 * H * Dh, torch.bfloat16)
    qkv.normal_()
    qkv.requires_grad_(True)
    meta = _meta(lens)
    o = qkv_attention(qkv, meta, H, H, Dh)
    o.backward(torch.randn_like(o))
    torch.cuda.synchronize()
    assert intact(big.detach(), T)
    assert bool(torch.isfinite(o).all())
