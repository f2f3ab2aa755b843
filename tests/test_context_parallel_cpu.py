"""Context parallelism, the pieces below the trainer: slicing a row inside documents and the differentiable gathers, on
three gloo ranks (one document spans all of them, so the prefix a rank borrows is longer than one slice)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flame_b200.ops.varlen import VarlenMeta
        from flame_b200.parallel.context_parallel import ContextParallel, borrow_prefix
        from flame_b200.ops.gla import gla, scalar_gla
        from flame_b200.ops import linear_attn as la
        T, per = 96, 32
        cu = torch.tensor([0, 10, 90, 96], dtype=torch.int32)       # the second document covers ranks 0, 1 and 2
        meta = VarlenMeta.from_cu_seqlens(cu, T, torch.device("cpu"))
        cp = ContextParallel.__new__(ContextParallel)
        cp.world, cp.rank, cp.group, cp.mode = world, rank, dist.group.WORLD, "sequence"
        ids = torch.arange(T).unsqueeze(0)
        _, _, lmeta = cp._slice_sequence(ids, ids.clone(), meta)
        sl = lmeta.sequence_slice
        assert sl.max_prefix == 54 and sl.continues == [False, True, True] and sl.single == [False, True, False]
        # borrow_prefix with a prefix longer than a slice: the whole-row gather
        x = (torch.arange(T, dtype=torch.float32)[:, None] * torch.ones(1, 3)).requires_grad_(True)
        mine = x[rank * per:(rank + 1) * per]
        (ext,) = borrow_prefix([mine], sl)
        lo = rank * per
        assert torch.equal(ext.detach()[:, 0], torch.arange(lo - sl.prefix, lo + per, dtype=torch.float32))
        ext.sum().backward()
        # a row is counted once by its owner and once by every later rank that borrowed it
        users = torch.zeros(T)
        for j in range(world):
            pj = [0, 22, 54][j]
            users[j * per - pj:(j + 1) * per] += 1
        assert torch.equal(x.grad[lo:lo + per, 0], users[lo:lo + per]), (rank, x.grad[lo:lo + per, 0], users[lo:lo + per])
        # state passing through a rank whose whole slice is the middle of one document (rank 1): gla and the scalar form
        torch.manual_seed(0)
        H, dk, dv = 2, 8, 4
        q, k, v = torch.randn(T, H, dk), torch.randn(T, H, dk), torch.randn(T, H, dv)
        g = torch.nn.functional.logsigmoid(torch.randn(T, H, dk))
        ref = la.gla_recurrent(q, k, v, g, meta, dk ** -0.5)
        got = gla(q[lo:lo + per], k[lo:lo + per], v[lo:lo + per], g[lo:lo + per], lmeta, dk ** -0.5)
        assert torch.allclose(got, ref[lo:lo + per], atol=2e-4), (rank, (got - ref[lo:lo + per]).abs().max())
        gs = torch.nn.functional.logsigmoid(torch.randn(T, H))
        ref2 = la.gla_recurrent(q, k, v, gs[..., None].expand(T, H, dk), meta, 1.0)
        got2 = scalar_gla(q[lo:lo + per], k[lo:lo + per], v[lo:lo + per], gs[lo:lo + per], lmeta, 1.0)
        assert torch.allclose(got2, ref2[lo:lo + per], atol=2e-4), (rank, (got2 - ref2[lo:lo + per]).abs().max())
        # the short convolution's halo rows, and the mixers that recompute a borrowed prefix, against the whole row
        from flame_b200.ops.conv import short_conv
        from flame_b200.ops.delta_rule import gated_delta_rule
        from flame_b200.ops.gla import gsa
        from flame_b200.ops.scan import selective_scan
        from flame_b200.ops.stickbreaking import sb_attention
        sl_ = slice(lo, lo + per)
        xc, wc, bc = torch.randn(T, 6), torch.randn(6, 1, 4), torch.randn(6)
        assert torch.allclose(short_conv(xc[sl_], wc, bc, lmeta, "silu"), short_conv(xc, wc, bc, meta, "silu")[sl_], atol=1e-5)
        beta, gd = torch.rand(T, H), -torch.rand(T, H) * 0.1
        vd = torch.randn(T, H, dv)
        ref3 = gated_delta_rule(q, k, vd, beta, gd, meta)
        got3 = gated_delta_rule(q[sl_], k[sl_], vd[sl_], beta[sl_], gd[sl_], lmeta)
        assert torch.allclose(got3, ref3[sl_], atol=2e-4), (rank, (got3 - ref3[sl_]).abs().max())
        slots = 4
        s_ = torch.rand(T, H, slots)
        gf = torch.nn.functional.logsigmoid(torch.randn(T, H, slots))
        ref4 = gsa(q, k, v, s_, gf, meta, dk ** -0.5)
        got4 = gsa(q[sl_], k[sl_], v[sl_], s_[sl_], gf[sl_], lmeta, dk ** -0.5)
        assert torch.allclose(got4, ref4[sl_], atol=2e-4), (rank, (got4 - ref4[sl_]).abs().max())
        Di, N = 6, 4
        u, dl = torch.randn(T, Di), torch.rand(T, Di) * 0.1
        A, Bm, Cm, Dm = -torch.rand(Di, N), torch.randn(T, N), torch.randn(T, N), torch.randn(Di)
        ref5 = selective_scan(u, dl, A, Bm, Cm, Dm, meta)
        got5 = selective_scan(u[sl_], dl[sl_], A, Bm[sl_], Cm[sl_], Dm, lmeta)
        assert torch.allclose(got5, ref5[sl_], atol=2e-4), (rank, (got5 - ref5[sl_]).abs().max())
        vs = torch.randn(T, H, dk)
        ref6, rem6 = sb_attention(q, k, vs, meta)
        got6, gotrem = sb_attention(q[sl_], k[sl_], vs[sl_], lmeta)
        assert torch.allclose(got6, ref6[sl_], atol=2e-4) and torch.allclose(gotrem, rem6[sl_], atol=2e-4)
        # gradients: the slices' losses summed over the ranks are the whole row's loss, so what reaches a rank's own rows
        # (its own contribution plus what later ranks send back through the gathers) must be the whole-row gradient
        os.environ["FLAME_B200_CP_DELTA"] = "state"

        def grads(fn_full, fn_slice, tensors):
            w_full = None
            leaves = [t.detach().clone().requires_grad_(True) for t in tensors]
            y = fn_full(*leaves)
            torch.manual_seed(123)
            w_full = torch.randn_like(y)
            (y * w_full).sum().backward()
            want = [l.grad[sl_].clone() for l in leaves]
            leaves2 = [t.detach().clone().requires_grad_(True) for t in tensors]
            y2 = fn_slice(*[l[sl_] for l in leaves2])
            (y2 * w_full[sl_]).sum().backward()
            got = [l.grad[sl_] for l in leaves2]
            for a_, b_ in zip(got, want):
                assert torch.allclose(a_, b_, atol=5e-4, rtol=1e-3), (rank, (a_ - b_).abs().max())

        grads(lambda q_, k_, v_, g_: la.gla_recurrent(q_, k_, v_, g_, meta, dk ** -0.5),
              lambda q_, k_, v_, g_: gla(q_, k_, v_, g_, lmeta, dk ** -0.5), [q, k, v, g])
        grads(lambda q_, k_, v_, b_, g_: gated_delta_rule(q_, k_, v_, b_, g_, meta),
              lambda q_, k_, v_, b_, g_: gated_delta_rule(q_, k_, v_, b_, g_, lmeta), [q, k, vd, beta, gd])
        grads(lambda q_, k_, v_, s2, g_: gsa(q_, k_, v_, s2, g_, meta, dk ** -0.5),
              lambda q_, k_, v_, s2, g_: gsa(q_, k_, v_, s2, g_, lmeta, dk ** -0.5), [q, k, v, s_, gf])
        grads(lambda u_, d_, b_, c_: selective_scan(u_, d_, A, b_, c_, Dm, meta),
              lambda u_, d_, b_, c_: selective_scan(u_, d_, A, b_, c_, Dm, lmeta), [u, dl, Bm, Cm])
        grads(lambda x_: short_conv(x_, wc, bc, meta, "silu"), lambda x_: short_conv(x_, wc, bc, lmeta, "silu"), [xc])
        grads(lambda q_, k_, v_: sb_attention(q_, k_, v_, meta)[0], lambda q_, k_, v_: sb_attention(q_, k_, v_, lmeta)[0],
              [q, k, vs])
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def test_slices_prefixes_and_state_chains_on_three_ranks():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(3, 29791, out), nprocs=3, join=True)
    assert dict(out) == {0: 1, 1: 1, 2: 1}
