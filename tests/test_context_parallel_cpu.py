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
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def test_slices_prefixes_and_state_chains_on_three_ranks():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(3, 29791, out), nprocs=3, join=True)
    assert dict(out) == {0: 1, 1: 1, 2: 1}
