"""Every model family learns on a GPU through the sharded engine and the CUDA kernels (``pytest -m gpu``): a small model
is stepped 30 times on one fixed packed batch and its loss must fall by a wide margin.  This exercises each family's
kernels, their gradients (including the special parameters A_log, dt_bias, D, convolution taps), the fp32-master AdamW
and gradient clipping end to end."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

FAMILIES = {
    "transformer": dict(num_heads=4),
    "sba": dict(num_heads=4),
    "gla": dict(num_heads=2, expand_k=0.5, expand_v=1.0),
    "hgrn2": dict(num_heads=2, expand_ratio=128),
    "gsa": dict(num_heads=2, num_slots=64),
    "delta_net": dict(num_heads=2),
    "gated_deltanet": dict(num_heads=2, head_dim=128),
    "mamba": dict(state_size=16),
    "mamba2": dict(head_dim=64, state_size=128, n_groups=1),
    "samba": dict(state_size=16, attn=dict(layers=[1], num_heads=4, num_kv_heads=4, qkv_bias=False, window_size=256,
                                           rope_theta=10000.0)),
}


@pytest.mark.parametrize("model_type", list(FAMILIES))
def test_family_overfits_a_fixed_batch_on_gpu(model_type):
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    torch.manual_seed(0)
    cfg = ModelConfig(model_type, hidden_size=256, num_hidden_layers=2, vocab_size=512, max_position_embeddings=4096,
                      **FAMILIES[model_type])
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device(DEV), torch.bfloat16,
                        OptimConfig(lr=3e-3, weight_decay=0.0, max_norm=1.0, skip_nan_inf=True))
    eng.init_weights(0)
    model.train()
    lens = [300, 77, 129, 1, 517]
    T = sum(lens)
    ids = torch.randint(3, 512, (1, T), device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
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
    assert all(l == l for l in losses), losses  # no NaN
    assert eng.skipped_steps() == 0
    assert losses[-1] < losses[0] - 1.5, (model_type, losses[0], losses[-1])
