"""Optimizer-state offload (``training.enable_cpu_offload``): same update, state in pinned host memory."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_offloaded_optimizer_matches_resident_optimizer():
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    cfg = ModelConfig("transformer", hidden_size=256, num_hidden_layers=3, vocab_size=512, max_position_embeddings=4096,
                      num_heads=4)
    lens = [120, 77, 128, 6]  # one key tile per document: no cross-CTA reduce-add, so the run is bitwise repeatable
    ids = torch.randint(3, 512, (1, sum(lens)), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    finals, losses = [], []
    for offload in (False, True):
        model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
        eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device("cuda"), torch.bfloat16,
                            OptimConfig(lr=3e-3, weight_decay=0.1, max_norm=1.0, skip_nan_inf=True), cpu_offload=offload)
        eng.init_weights(0)
        model.train()
        assert eng.units[0].master.is_cuda != offload
        if offload:
            assert eng.units[0].master.is_pinned() and eng.units[0].exp_avg_sq.is_pinned()
        run = []
        for _ in range(4):
            eng.zero_grad()
            out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
            out.loss.backward()
            eng.step(3e-3)
            run.append(float(out.loss.detach()))
        torch.cuda.synchronize()
        assert eng.applied_steps() == 4
        finals.append([u.master.detach().cpu().clone() for u in eng.units] + [eng.compute_all.detach().cpu().clone()])
        losses.append(run)
        state = eng.full_state("exp_avg")
        assert all(torch.isfinite(v).all() for v in state.values())
    assert losses[0] == losses[1]
    for a, b in zip(*finals):
        assert torch.equal(a, b)   # same kernels on the same values: bitwise identical


def test_activation_offload_round_trip_matches_plain_training():
    """Saved activations go to pinned host memory on a side stream and come back (prefetched) in backward: same losses,
    a bounded forward stash, the head exempted."""
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    from flame_b200.parallel.activation_offload import enable_activation_offload
    from flame_b200.parallel.parallelize import Runner
    cfg = ModelConfig("transformer", hidden_size=256, num_hidden_layers=3, vocab_size=512, max_position_embeddings=4096,
                      num_heads=4)
    lens = [120, 77, 128, 59]
    ids = torch.randint(3, 512, (1, sum(lens)), generator=torch.Generator().manual_seed(1))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    batch = {"input_ids": ids, "labels": ids.clone(), "cu_seqlens": cu}
    curves, ctxs = [], []
    for offload in (False, True):
        model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
        dims = ParallelDims(world_size=1)
        eng = ShardedEngine(model, dims, torch.device("cuda"), torch.bfloat16, OptimConfig(lr=3e-3))
        eng.init_weights(0)
        model.train()
        runner = Runner(model, eng, dims, torch.device("cuda"))
        ctx = enable_activation_offload(runner, max_fwd_stash_size=3) if offload else None
        run = []
        for _ in range(3):
            eng.zero_grad()
            loss = runner.forward_backward(batch, 1.0)
            eng.step(3e-3)
            run.append(float(loss))
        curves.append(run)
        ctxs.append(ctx)
    # a tensor that comes back from the host is contiguous, where the original may have been a column block of a fused
    # buffer, so a few products take another (equally valid) path: equal to rounding, not bit for bit
    assert curves[0][0] == curves[1][0]
    for a, b in zip(curves[0], curves[1]):
        assert abs(a - b) < 1e-4 * abs(a), (curves[0], curves[1])
    ctx = ctxs[1]
    assert ctx.offloaded_tensors > 10 and ctx.offloaded_bytes > 1 << 20
    assert ctx.max_stash_seen <= 3 and ctx.prefetched > 0
    assert not ctx.records and model.head_saved_tensors_ctx is not None   # everything came back; the head is exempt


def test_noop_manager_switches_outer_hooks_off():
    from flame_b200.parallel.activation_offload import NoOpManager
    seen = []

    def pack(t):
        seen.append(t.shape)
        return t

    x = torch.randn(8, 8, device="cuda", requires_grad=True)
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        y = (x * x).sum()
        n_outer = len(seen)
        with NoOpManager():
            z = (x * x).sum()
        assert len(seen) == n_outer and n_outer > 0
    (y + z).backward()
