"""``AutoConfig`` / ``AutoModelForCausalLM`` registration (custom_models/sba/__init__.py:1-9 in the reference)."""
import pytest
import torch


def test_saved_model_loads_through_the_auto_classes(tmp_path):
    transformers = pytest.importorskip("transformers")
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.models.hf import register
    done = register(["sba"])
    assert done in (["sba"], [])  # [] when an earlier test registered it already
    cfg = ModelConfig("sba", hidden_size=64, num_hidden_layers=2, num_heads=2, vocab_size=128)
    ours = build_model(cfg, device="cpu", dtype=torch.float32, init=True, seed=3)
    ours.eval()
    ours.save_pretrained(str(tmp_path))
    conf = transformers.AutoConfig.from_pretrained(str(tmp_path))
    assert conf.model_type == "sba" and conf.hidden_size == 64 and conf.num_hidden_layers == 2
    theirs = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path))
    theirs.eval()
    a, b = ours.state_dict(), theirs.state_dict()
    assert set(a) == set(b)
    for k in a:
        assert torch.equal(a[k], b[k].to(a[k].dtype)), k
    ids = torch.randint(3, 128, (2, 24), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        lo = ours(input_ids=ids, labels=ids, return_logits=True)
        lt = theirs(input_ids=ids, labels=ids)
    assert torch.allclose(lo.loss, lt.loss, atol=1e-5) and torch.allclose(lo.logits, lt.logits, atol=1e-4)
    # and back: what the Auto class saves, this package loads
    out2 = tmp_path / "resaved"
    theirs.save_pretrained(str(out2))
    from flame_b200.models import CausalLM
    again = CausalLM.from_pretrained(str(out2))
    for k, v in again.state_dict().items():
        assert torch.equal(v, a[k]), k
