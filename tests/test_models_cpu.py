"""Every model family builds from its shipped JSON with the reference's state-dict names and trains on CPU."""
import glob
import os

import pytest
import torch

from flame_b200.models import ModelConfig, build_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# parameter totals of the reference models built from the same JSON files
EXPECTED_PARAMS = {
    "transformer_340M": 373.9e6, "sba_340m": 373.9e6, "gla_340M": 374.5e6, "delta_net_340M": 374.4e6,
    "gated_deltanet_340M": 512.3e6, "gsa_340M": 380.2e6, "hgrn2_340M": 373.9e6, "mamba_340M": 385.6e6,
    "mamba2_340M": 382.4e6, "samba_1B": 1.404e9, "gated_deltanet_1B": 1.387e9, "gla_7B": 6.742e9,
    "transformer_7B": 7.242e9, "transformer_1B": 1.364e9, "delta_net_1B": 1.366e9, "gsa_1B": 1.377e9,
    "mamba_1B": 1.400e9, "mamba2_1B": 1.372e9,
}


@pytest.mark.parametrize("name", sorted(EXPECTED_PARAMS))
def test_parameter_counts_match_reference(name):
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", name + ".json"))
    model = build_model(cfg, device="meta", init=False)
    n = model.num_parameters()
    assert abs(n - EXPECTED_PARAMS[name]) / EXPECTED_PARAMS[name] < 2e-3, (name, n)


def test_state_dict_names_follow_reference_layout():
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", "gated_deltanet_1B.json"))
    sd = build_model(cfg, device="meta", init=False).state_dict()
    assert sd["model.layers.0.attn.A_log"].shape == (6,)
    assert sd["model.layers.0.attn.q_proj.weight"].shape == (1536, 2048)
    assert sd["model.layers.0.attn.v_conv1d.weight"].shape == (3072, 1, 4)
    assert sd["model.layers.0.attn.o_norm.weight"].shape == (512,)
    assert sd["model.layers.3.mlp.down_proj.weight"].shape == (2048, 5632)
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", "mamba2_340M.json"))
    sd = build_model(cfg, device="meta", init=False).state_dict()
    assert sd["backbone.layers.0.mixer.in_proj.weight"].shape == (4384, 1024)
    assert sd["backbone.layers.0.mixer.conv1d.weight"].shape == (2304, 1, 4)
    assert sd["backbone.norm_f.weight"].shape == (1024,)
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", "gla_340M.json"))
    sd = build_model(cfg, device="meta", init=False).state_dict()
    assert sd["model.layers.0.attn.gk_proj.1.bias"].shape == (512,)
    assert sd["model.layers.0.attn.g_norm_swish_gate.weight"].shape == (256,)
    cfg = ModelConfig.from_pretrained(os.path.join(ROOT, "configs", "hgrn2_340M.json"))
    sd = build_model(cfg, device="meta", init=False).state_dict()
    assert sd["model.lower_bounds"].shape == (24, 1024)


def _tiny(model_type, **kw):
    base = dict(hidden_size=64, num_hidden_layers=2, vocab_size=128, max_position_embeddings=256)
    per = {
        "transformer": dict(num_heads=4), "sba": dict(num_heads=4), "gla": dict(num_heads=2),
        "delta_net": dict(num_heads=2), "gated_deltanet": dict(num_heads=2, head_dim=16),
        "gsa": dict(num_heads=2, num_slots=8), "hgrn2": dict(num_heads=2, expand_ratio=32),
        "mamba": dict(state_size=4), "mamba2": dict(head_dim=16, state_size=8),
        "samba": dict(state_size=4, intermediate_size=128, time_step_rank=4,
                      attn=dict(layers=[1], num_heads=4, num_kv_heads=4, qkv_bias=False, window_size=16, rope_theta=10000.0)),
    }
    base.update(per[model_type])
    base.update(kw)
    return ModelConfig(model_type, **base)


@pytest.mark.parametrize("model_type", ["transformer", "sba", "gla", "delta_net", "gated_deltanet", "gsa", "hgrn2",
                                        "mamba", "mamba2", "samba"])
def test_tiny_model_trains_on_cpu(model_type):
    torch.manual_seed(0)
    cfg = _tiny(model_type)
    model = build_model(cfg, seed=1)
    ids = torch.randint(3, 128, (1, 96))
    cu = torch.tensor([0, 40, 41, 96], dtype=torch.int32)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
        opt.zero_grad()
        out.loss.backward()
        opt.step()
        losses.append(out.loss.item())
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0]


def test_packed_documents_do_not_leak(tmp_path):
    """Changing document 0 must not change the hidden states of document 1."""
    for mt in ["transformer", "gla", "gated_deltanet", "mamba2", "mamba", "sba"]:
        cfg = _tiny(mt)
        model = build_model(cfg, seed=2).eval()
        ids = torch.randint(3, 128, (1, 64))
        ids2 = ids.clone()
        ids2[0, :20] = torch.randint(3, 128, (20,))
        cu = torch.tensor([0, 20, 64], dtype=torch.int32)
        with torch.no_grad():
            a = model(input_ids=ids, cu_seqlens=cu).logits
            b = model(input_ids=ids2, cu_seqlens=cu).logits
        assert torch.allclose(a[20:], b[20:], atol=1e-5), mt
        assert not torch.allclose(a[:20], b[:20], atol=1e-5), mt


def test_save_and_load_pretrained_roundtrip(tmp_path):
    cfg = _tiny("gla")
    model = build_model(cfg, seed=3)
    model.save_pretrained(str(tmp_path / "hf"))
    from flame_b200.models import CausalLM
    again = CausalLM.from_pretrained(str(tmp_path / "hf"))
    for (k1, v1), (k2, v2) in zip(model.state_dict().items(), again.state_dict().items()):
        assert k1 == k2 and torch.equal(v1, v2)
