"""Operator-level selective activation checkpointing (``--activation_checkpoint.selective_ac_option op``) on CPU:
the recomputation replays kept matrix products instead of running them, and gradients equal the unchecked model's."""
import torch

from flame_b200.models import ModelConfig, build_model
from flame_b200.ops import sac
from flame_b200.parallel.parallelize import apply_activation_checkpointing


def _model(seed=0):
    cfg = ModelConfig("transformer", hidden_size=64, num_hidden_layers=2, num_heads=2, vocab_size=128)
    m = build_model(cfg, device="cpu", dtype=torch.float32, init=False)
    m.init_weights(seed)
    m.train()
    return m


def test_tape_policy_keeps_every_other_product_and_all_attention():
    t = sac.Tape()
    t.begin_run()
    assert t.mode == "record"
    kept = []
    for kind in ["mm", "attn", "mm", "mm", "mm"]:
        keep = t.decide(kind)
        kept.append(keep)
        t.store(torch.ones(2))
    assert kept == [True, True, False, True, False]
    t.begin_run()
    assert t.mode == "replay"
    got = [t.fetch() is not None for _ in range(5)]
    assert got == kept
    assert t.fetch() is None and t.kept_bytes() == 0   # past the end: recompute; fetched values were released


def test_selective_op_checkpointing_matches_plain_backward(monkeypatch):
    ids = torch.randint(3, 128, (2, 48), generator=torch.Generator().manual_seed(1))
    plain, ckpt = _model(), _model()
    apply_activation_checkpointing(ckpt, "selective", "op")
    from flame_b200.ops import linear as linear_mod
    calls = {"n": 0}
    real = linear_mod.gemm_nt

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    lp = plain(input_ids=ids, labels=ids).loss
    lp.backward()
    monkeypatch.setattr(linear_mod, "gemm_nt", counting)
    lc = ckpt(input_ids=ids, labels=ids).loss
    fwd_calls = calls["n"]
    lc.backward()
    recompute_calls = calls["n"] - fwd_calls
    assert torch.allclose(lp, lc)
    for (n, a), (_, b) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert a.grad is not None and torch.allclose(a.grad, b.grad, atol=1e-6), n
    # each block has 4 products (qkv, o, gate|up, down; 7 GEMM launches without the engine's fused weight layout): the
    # 1st and 3rd are replayed from the tape, the 2nd and 4th (one launch each) are recomputed
    assert fwd_calls == 14 and recompute_calls == 4, (fwd_calls, recompute_calls)


def test_invalid_selective_option_is_an_error():
    import pytest
    with pytest.raises(ValueError, match="Invalid selective AC option"):
        apply_activation_checkpointing(_model(), "selective", "sometimes")


def test_mixer_recompute_keeps_gradients_and_saves_less():
    """``selective_ac_option mixer``: the chunk pipeline of a token mixer is run again in backward; same gradients."""
    import torch
    from flame_b200.ops import chunked
    from flame_b200.ops.varlen import VarlenMeta
    torch.manual_seed(0)
    T, H, dk, dv = 200, 2, 16, 32
    cu = torch.tensor([0, 70, 200], dtype=torch.int32)
    meta = VarlenMeta.from_cu_seqlens(cu, T, torch.device("cpu"))

    def run(flag):
        chunked.set_mixer_recompute(flag)
        try:
            torch.manual_seed(1)
            q = torch.nn.functional.normalize(torch.randn(T, H, dk), dim=-1).requires_grad_(True)
            k = torch.nn.functional.normalize(torch.randn(T, H, dk), dim=-1).requires_grad_(True)
            v = torch.randn(T, H, dv, requires_grad=True)
            beta = torch.rand(T, H, requires_grad=True)
            g = (-torch.rand(T, H) * 0.1).requires_grad_(True)
            saved = []
            with torch.autograd.graph.saved_tensors_hooks(lambda t: (saved.append(t.numel()), t)[1], lambda t: t):
                o = chunked.gated_delta_rule_tc(q, k, v, beta, g, meta)
            o.square().sum().backward()
            return o.detach(), [t.grad.clone() for t in (q, k, v, beta, g)], sum(saved)
        finally:
            chunked.set_mixer_recompute(False)

    o0, g0, n0 = run(False)
    o1, g1, n1 = run(True)
    assert torch.allclose(o0, o1, atol=1e-6)
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
    assert n1 < n0 / 3, (n0, n1)
