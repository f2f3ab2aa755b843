"""Operator micro-benchmarks and roofline fractions for the kernel library.

    python -m flame_b200.tools.opbench gemm                 # tcgen05 GEMM vs torch.matmul on the training shapes
    python -m flame_b200.tools.opbench attention            # varlen attention fwd / bwd (+ flash-attn if importable)
    python -m flame_b200.tools.opbench elementwise          # norm / swiglu / rope / cross-entropy / adamw bandwidth
    python -m flame_b200.tools.opbench mixers               # chunked delta rule / GLA / SSD fwd and fwd+bwd
    python -m flame_b200.tools.opbench scan                 # Mamba-1 selective scan fwd and fwd+bwd
    python -m flame_b200.tools.opbench step [--tokens N]    # one training step of transformer_340M (for ncu captures)

Timing: CUDA events on the launching stream after warm-up, a 256 MiB buffer is rewritten before every timed
iteration (L2 flush).  Fractions are reported against the peaks in ``MEASURED_PEAKS.json`` at the repository root
when that file exists ("of measured"), else against 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


_FLUSH = None


def timeit(fn, iters: int = 10, warmup: int = 3) -> float:
    """Median milliseconds per call, L2 flushed before each timed call."""
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _FLUSH.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def synthetic_meta(T: int, lo: int = 64, hi: int = 4096, seed: int = 0):
    from flame_b200.ops.varlen import VarlenMeta
    rng = random.Random(seed)
    lens, tot = [], 0
    while tot < T:
        l = min(rng.randint(lo, hi), T - tot)
        lens.append(l)
        tot += l
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return VarlenMeta.from_cu_seqlens(cu, T, torch.device("cuda")), lens


def bench_gemm(args) -> None:
    from flame_b200.ops import gemm
    _, peak, tag = peaks()
    dev = "cuda"
    print(f"bf16 GEMM, fraction {tag} ({peak / 1e12:.0f} TFLOP/s)")
    shapes = [(65536, 3072, 1024), (65536, 1024, 1024), (65536, 5632, 1024), (65536, 1024, 2816), (8192, 8192, 8192),
              (8192, 32000, 1024)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        t1 = timeit(lambda: gemm.gemm_nt(a, b, out=out, splits=1))
        t2 = timeit(lambda: torch.matmul(a, b.t(), out=out))
        print(f"  nt {M}x{N}x{K}: {t1:.3f} ms {fl / t1 / 1e9:7.0f} TF ({fl / t1 / 1e-3 / peak:.2f}) | torch.matmul {t2:.3f} ms "
              f"{fl / t2 / 1e9:7.0f} TF")
        bt = b.t().contiguous()
        t1 = timeit(lambda: gemm.gemm_nn(a, bt, out=out, splits=1))
        print(f"  nn {M}x{N}x{K}: {t1:.3f} ms {fl / t1 / 1e9:7.0f} TF ({fl / t1 / 1e-3 / peak:.2f})")
    for T, N, K in [(65536, 3072, 1024), (65536, 1024, 1024), (65536, 5632, 1024), (65536, 1024, 2816)]:
        dy = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(N, K, device=dev, dtype=torch.float32)
        fl = 2.0 * T * N * K
        t1 = timeit(lambda: gemm.gemm_tn(dy, x, out=out, accumulate=True))
        o2 = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        t2 = timeit(lambda: torch.matmul(dy.t(), x, out=o2))
        print(f"  tn(wgrad, fp32 accumulate) {T}x{N}x{K}: {t1:.3f} ms {fl / t1 / 1e9:7.0f} TF ({fl / t1 / 1e-3 / peak:.2f}) | "
              f"torch.matmul {t2:.3f} ms {fl / t2 / 1e9:7.0f} TF")


def bench_fp8(args) -> None:
    """fp8 GEMM (kind::f8f6f4) and a whole Float8 linear layer (quantisation included) against the bf16 layer."""
    from flame_b200.ops import float8, gemm
    _, peak, tag = peaks()
    dev = "cuda"
    print(f"fp8 GEMM (e4m3 x e4m3, bf16 out); fraction of the bf16 peak {tag} ({peak / 1e12:.0f} TFLOP/s)")
    for M, N, K in [(65536, 3072, 1024), (65536, 1024, 2816), (8192, 8192, 8192), (16384, 16384, 4096)]:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        aq, _, ai = float8.quantize(a, transpose=False)
        bq, _, bi = float8.quantize(b, transpose=False)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        t8 = timeit(lambda: float8.gemm_fp8(aq, bq, ai, bi, out=out))
        t16 = timeit(lambda: gemm.gemm_nt(a, b, out=out, splits=1))
        tq = timeit(lambda: float8.quantize(a, transpose=True))
        gb = M * K * 4 / tq / 1e6
        print(f"  {M}x{N}x{K}: fp8 {t8:.3f} ms {fl / t8 / 1e9:7.0f} TF ({fl / t8 / 1e-3 / peak:.2f}) | bf16 {t16:.3f} ms "
              f"{fl / t16 / 1e9:7.0f} TF | quantize A (+transpose) {tq:.3f} ms {gb:6.0f} GB/s")
    from flame_b200.ops.linear import linear
    for T, N, K in [(65536, 3072, 1024), (65536, 2816 * 2, 1024), (16384, 3 * 4096, 4096), (16384, 2 * 11008, 4096)]:
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16, requires_grad=True)
        g = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
        res = {}
        for tag8 in (False, True):
            w = torch.nn.Parameter(torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02)
            w.main_grad = torch.zeros(N, K, device=dev)
            if tag8:
                w._fp8 = True

            def fb():
                y = linear(x, w)
                y.backward(g)
                x.grad = None
            res[tag8] = timeit(fb)
        print(f"  linear fwd+bwd {T}x{N}x{K}: bf16 {res[False]:.3f} ms | float8 (casts included) {res[True]:.3f} ms "
              f"({res[False] / res[True]:.2f}x)")


def bench_attention(args) -> None:
    from flame_b200.ops.attention import attention
    _, peak, tag = peaks()
    T, H, Dh = args.tokens, args.heads, args.head_dim
    meta, lens = synthetic_meta(T)
    qkv = torch.randn(T, 3 * H * Dh, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, :H * Dh].view(T, H, Dh).detach().requires_grad_(True)
    k = qkv[:, H * Dh:2 * H * Dh].view(T, H, Dh).detach().requires_grad_(True)
    v = qkv[:, 2 * H * Dh:].view(T, H, Dh).detach().requires_grad_(True)
    fl = sum(4.0 * l * l / 2 * H * Dh for l in lens)
    t_f = timeit(lambda: attention(q, k, v, meta))
    o = attention(q, k, v, meta)
    do = torch.randn_like(o)

    def fb():
        q.grad = k.grad = v.grad = None
        attention(q, k, v, meta).backward(do)

    t_fb = timeit(fb)
    print(f"varlen causal attention, T={T} H={H} Dh={Dh}, docs 64..4096; causal FLOPs; fraction {tag}")
    print(f"  fwd      {t_f:.3f} ms  {fl / t_f / 1e9:6.0f} TF ({fl / t_f / 1e-3 / peak:.2f})")
    print(f"  fwd+bwd  {t_fb:.3f} ms; bwd {t_fb - t_f:.3f} ms {2.5 * fl / (t_fb - t_f) / 1e9:6.0f} TF "
          f"({2.5 * fl / (t_fb - t_f) / 1e-3 / peak:.2f})")
    try:
        from flash_attn import flash_attn_varlen_func
        cu = meta.cu_seqlens
        qq, kk, vv = (x.detach().contiguous().requires_grad_(True) for x in (q, k, v))
        t3 = timeit(lambda: flash_attn_varlen_func(qq, kk, vv, cu, cu, 4096, 4096, causal=True))

        def fb2():
            qq.grad = kk.grad = vv.grad = None
            flash_attn_varlen_func(qq, kk, vv, cu, cu, 4096, 4096, causal=True).backward(do)

        t4 = timeit(fb2)
        print(f"  flash-attn 2: fwd {t3:.3f} ms {fl / t3 / 1e9:6.0f} TF; bwd {t4 - t3:.3f} ms {2.5 * fl / (t4 - t3) / 1e9:6.0f} TF")
    except Exception as e:
        print(f"  flash-attn comparison unavailable: {e!r}")


def bench_elementwise(args) -> None:
    from flame_b200.ops import optim as O
    from flame_b200.ops.activations import swiglu
    from flame_b200.ops.cross_entropy import cross_entropy
    from flame_b200.ops.norm import rms_norm
    bw, _, tag = peaks()
    T, D, I = args.tokens, 1024, 2816
    print(f"bandwidth-bound kernels, T={T}; achieved GB/s over algorithmic bytes; fraction {tag} ({bw / 1e9:.0f} GB/s)")

    def report(name, ms, nbytes):
        print(f"  {name:34s} {ms:.3f} ms  {nbytes / ms / 1e6:7.0f} GB/s ({nbytes / ms / 1e-3 / bw:.2f})")

    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    report("rmsnorm fwd (+residual, prenorm)", timeit(lambda: rms_norm(x, w, 1e-6, r, True)), 4 * T * D * 2)
    y, res = rms_norm(x, w, 1e-6, r, True)
    gy, gr = torch.randn_like(y), torch.randn_like(res)
    report("rmsnorm bwd (+residual grad)", timeit(lambda: torch.autograd.grad([y, res], [x, r, w], [gy, gr], retain_graph=True)),
           4 * T * D * 2)
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    report("swiglu fwd", timeit(lambda: swiglu(gu)), 3 * T * I * 2)
    a = swiglu(gu)
    da = torch.randn_like(a)
    report("swiglu bwd", timeit(lambda: torch.autograd.grad(a, gu, da, retain_graph=True)), 5 * T * I * 2)
    V, Tc = 32000, 8192
    lab = torch.randint(0, V, (Tc,), device="cuda")
    base = torch.randn(Tc, V, device="cuda", dtype=torch.bfloat16)
    report("cross-entropy fwd+grad (in place)", timeit(lambda: cross_entropy(base.clone().requires_grad_(True), lab)) -
           timeit(lambda: base.clone()), 3 * Tc * V * 2)
    n = 64 << 20
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ctrl = torch.zeros(O.CTRL_SIZE, device="cuda")
    ctrl[0] = 1.0
    report("adamw (fp32 master, bf16 out)", timeit(lambda: O.adamw_step(p, m, v, g, lp, ctrl, 1e-4, .9, .95, 1e-8, .1, 1., True)),
           n * (4 * 4 + 3 * 4 + 2))


def bench_swiglu(args) -> None:
    """gate | up projection + SwiGLU: the GEMM with the activation in its epilogue against GEMM + elementwise kernel."""
    from flame_b200.ops import activations, linear as linear_ops
    _, peak, tag = peaks()
    T, D, I = args.tokens, 1024, 2816
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(2 * I, D, device="cuda", dtype=torch.bfloat16) * 0.02)
    wg, wu = w[:I].detach().requires_grad_(True), w[I:].detach().requires_grad_(True)
    wg.data, wu.data = w[:I], w[I:]   # adjacent in memory, like the parameters of a unit
    dz = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * T * 2 * I * D

    os.environ["FLAME_B200_FUSED_SWIGLU"] = "1"   # opt-in: see ops/linear.py

    def fused():
        return linear_ops.gate_up_swiglu(x, wg, wu)

    def unfused():
        return activations.swiglu(linear_ops.linear_fused(x, [wg, wu]))

    for name, fn in (("GEMM with SwiGLU epilogue", fused), ("GEMM + swiglu kernel", unfused)):
        def nograd():
            with torch.no_grad():
                return fn()
        f = timeit(nograd, iters=args.iters)

        def fb():
            x.grad = wg.grad = wu.grad = None
            fn().backward(dz)
        b = timeit(fb, iters=args.iters)
        print(f"  {name:28s} fwd {f:.3f} ms ({fl / f / 1e9:5.0f} TF, {fl / f / 1e-3 / peak:.2f} {tag})   fwd+bwd {b:.3f} ms")


def bench_mixers(args) -> None:
    """Forward + backward of the chunk-parallel token mixers at the shapes of the configs in ``configs/``."""
    from flame_b200.ops import _lib
    from flame_b200.ops.chunk_kernels import l2norm
    from flame_b200.ops.chunked import gated_delta_rule_tc, gla_tc, scalar_gla_tc
    T = args.tokens
    meta, lens = synthetic_meta(T, 256, 4096)
    dev = "cuda"

    def leaf(*shape, dtype=torch.bfloat16):
        return torch.randn(*shape, device=dev, dtype=dtype).requires_grad_(True)

    def report(name, fn, do, flops):
        def nograd():
            with torch.no_grad():
                return fn()
        f, b = timeit(nograd, iters=args.iters), timeit(lambda: fn().backward(do), iters=args.iters)
        print(f"  {name:40s} fwd {f:7.3f} ms   fwd+bwd {b:7.3f} ms   ({flops / f / 1e9:6.1f} TFLOP/s algorithmic, fwd)", flush=True)

    print(f"token mixers, {T} packed tokens in {len(lens)} documents (<= 4096)")
    # ---- gated delta rule, gated_deltanet_1B: 6 heads, dk 256, dv 512
    H, dk, dv = 6, 256, 512
    q, k, v = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv)
    beta = torch.rand(T, H, device=dev).requires_grad_(True)
    g = (-torch.rand(T, H, device=dev) * 0.1).requires_grad_(True)
    do = torch.randn(T, H, dv, device=dev, dtype=torch.bfloat16)
    # per token and head: scores 2*2*64*dk, WY 2*64*(dk+dv), state 4*dk*dv, outputs 2*dk*dv + 2*64*dv + 2*dk*dv
    fl = T * H * (4 * 64 * dk + 2 * 64 * (dk + dv) + 8 * dk * dv + 2 * 64 * dv)
    report("gated delta rule  H6 dk256 dv512", lambda: gated_delta_rule_tc(l2norm(q), l2norm(k), v, beta, g, meta), do, fl)
    # ---- GLA, gla_340M: 4 heads, dk 128, dv 256
    H, dk, dv = 4, 128, 256
    q, k, v = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv)
    gk = torch.nn.functional.logsigmoid(torch.randn(T, H, dk, device=dev)).div(16).requires_grad_(True)
    do = torch.randn(T, H, dv, device=dev, dtype=torch.bfloat16)
    fl = T * H * (2 * 64 * dk + 4 * dk * dv + 2 * 64 * dv)
    report("GLA  H4 dk128 dv256", lambda: gla_tc(q, k, v, gk, meta), do, fl)
    # ---- Mamba2 SSD, mamba2_340M-like: 32 heads, state 128, head dim 64
    H, dk, dv = 32, 128, 64
    q, k, v = leaf(T, H, dk), leaf(T, H, dk), leaf(T, H, dv)
    g = (-torch.rand(T, H, device=dev) * 0.1).requires_grad_(True)
    do = torch.randn(T, H, dv, device=dev, dtype=torch.bfloat16)
    fl = T * H * (2 * 64 * dk + 4 * dk * dv + 2 * 64 * dv)
    report("scalar-gated (SSD)  H32 N128 P64", lambda: scalar_gla_tc(q, k, v, g, meta, 1.0), do, fl)
    _lib.assert_status_ok()


def bench_scan(args) -> None:
    """Mamba-1 selective scan forward / forward+backward at the mamba_340M shapes (Di 2048, N 16)."""
    from flame_b200.ops import _lib
    from flame_b200.ops.scan import selective_scan
    hbm, _, tag = peaks()
    T, Di, N = args.tokens, 2048, 16
    meta, lens = synthetic_meta(T, 256, 4096)
    dev = "cuda"
    u = torch.randn(T, Di, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    delta = (torch.rand(T, Di, device=dev) * 0.1).requires_grad_(True)
    A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32)[None].repeat(Di, 1).requires_grad_(True)
    B = torch.randn(T, N, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    C = torch.randn(T, N, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    D = torch.ones(Di, device=dev).requires_grad_(True)
    dy = torch.randn(T, Di, device=dev, dtype=torch.bfloat16)

    def fwd():
        with torch.no_grad():
            return selective_scan(u, delta, A, B, C, D, meta)

    def fb():
        selective_scan(u, delta, A, B, C, D, meta).backward(dy)
    f, b = timeit(fwd, iters=args.iters), timeit(fb, iters=args.iters)
    steps = T * Di * N
    print(f"selective scan, T={T} Di={Di} N={N}, {len(lens)} documents: fwd {f:.3f} ms, fwd+bwd {b:.3f} ms "
          f"({2 * steps / f / 1e6:.0f} G state updates/s forward incl. the two sweeps)")
    _lib.assert_status_ok()


def bench_step(args) -> None:
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    dev = torch.device("cuda:0")
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", args.model + ".json"))
    if args.layers:
        cfg.num_hidden_layers = args.layers
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), dev, torch.bfloat16, OptimConfig(lr=3e-4, eps=1e-15, skip_nan_inf=True))
    eng.init_weights(42)
    model.train()
    meta, _ = synthetic_meta(args.tokens)
    ids = torch.randint(3, 32000, (1, args.tokens), device=dev)

    def step():
        eng.zero_grad()
        out = model(input_ids=ids, labels=ids, meta=meta)
        out.loss.backward()
        eng.step(3e-4)

    ms = timeit(step, iters=args.iters, warmup=2)
    _lib.assert_status_ok()
    print(f"{args.model} ({cfg.num_hidden_layers} layers) one training step at {args.tokens} tokens: {ms:.2f} ms, "
          f"{args.tokens / ms * 1e3:,.0f} tokens/s")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "fp8", "attention", "elementwise", "swiglu", "mixers", "scan", "step"])
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--model", default="transformer_340M")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=64)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    {"gemm": bench_gemm, "fp8": bench_fp8, "attention": bench_attention, "elementwise": bench_elementwise, "swiglu": bench_swiglu, "mixers": bench_mixers,
     "scan": bench_scan, "step": bench_step}[args.what](args)


if __name__ == "__main__":
    main()
