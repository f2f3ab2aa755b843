"""DCP checkpoint -> HF directory -> DCP step-0 -> trainer resume (CPU)."""
import json
import os

import torch

from test_trainer_cpu import TINY, _args


def test_dcp_to_hf_and_back(tmp_path):
    from flame_b200.config_manager import JobConfig
    from flame_b200.models import CausalLM
    from flame_b200.train import main
    from flame_b200.utils.convert_dcp_to_hf import save_pretrained
    from flame_b200.utils.convert_hf_to_dcp import convert_hf_weights
    tmp = str(tmp_path)
    args = _args(tmp, steps=3, extra=["--checkpoint.enable_checkpoint", "--checkpoint.interval", "3"])
    main(JobConfig().parse_args(args))
    exp = os.path.join(tmp, "exp")
    save_pretrained(exp, 3, os.path.join(tmp, "tiny.json"))
    assert os.path.isfile(os.path.join(exp, "model.safetensors")) and os.path.isfile(os.path.join(exp, "config.json"))
    model = CausalLM.from_pretrained(exp)
    assert model.model.layers[1].mlp.down_proj.weight.shape == (256, 688)
    # HF -> DCP step-0 in a fresh run folder; the trainer loads only the model from a step-0 checkpoint
    exp2 = os.path.join(tmp, "exp2")
    convert_hf_weights(exp, os.path.join(exp2, "checkpoint", "step-0"))
    a2 = [x if x != exp else exp2 for x in _args(tmp, steps=1, extra=["--checkpoint.enable_checkpoint", "--checkpoint.interval",
                                                                     "100", "--checkpoint.load_step", "0"])]
    state = main(JobConfig().parse_args(a2))
    assert state.step == 1
    # the loss right after loading trained weights is lower than a cold start's first loss
    os.makedirs(os.path.join(tmp, "cold"), exist_ok=True)
    cold = main(JobConfig().parse_args(_args(os.path.join(tmp, "cold"), steps=1)))
    assert state.global_avg_losses[0] < cold.global_avg_losses[0]


def test_keep_latest_k_and_async_mode(tmp_path):
    from flame_b200.config_manager import JobConfig
    from flame_b200.train import main
    tmp = str(tmp_path)
    args = _args(tmp, steps=6, extra=["--checkpoint.enable_checkpoint", "--checkpoint.interval", "2",
                                      "--checkpoint.keep_latest_k", "2", "--checkpoint.async_mode", "async"])
    main(JobConfig().parse_args(args))
    steps = sorted(os.listdir(os.path.join(tmp, "exp", "checkpoint")))
    assert steps == ["step-4", "step-6"], steps


# ---------------------------------------------------------------------------------------------------------------
# interchange with the reference's own converter scripts (installed, unmodified, under baseline/_ref)
# ---------------------------------------------------------------------------------------------------------------
def _reference_tools():
    import importlib
    import sys
    import types
    ref = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "flame")):
        import pytest
        pytest.skip("the reference is not installed under baseline/_ref")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    # the reference's converter imports a namespace package of its source tree only for its side effects
    sys.modules.setdefault("custom_models", types.ModuleType("custom_models"))
    return (importlib.import_module("flame.utils.convert_dcp_to_hf"), importlib.import_module("flame.utils.convert_hf_to_dcp"))


def test_checkpoints_interchange_with_the_reference_converters(tmp_path):
    """(1) A checkpoint written by this trainer goes through the reference's ``convert_dcp_to_hf`` into an ``fla`` model
    whose weights equal ours.  (2) An ``fla`` model written by the reference's ``convert_hf_to_dcp`` as ``step-0`` is
    loaded by this trainer's checkpoint manager."""
    import pathlib
    import torch.distributed.checkpoint as dcp
    from flame_b200.config_manager import JobConfig
    from flame_b200.models import CausalLM, ModelConfig, build_model
    from flame_b200.train import main
    to_hf, to_dcp = _reference_tools()
    tmp = str(tmp_path)
    args = _args(tmp, steps=2, extra=["--checkpoint.enable_checkpoint", "--checkpoint.interval", "2"])
    main(JobConfig().parse_args(args))
    exp = os.path.join(tmp, "exp")
    meta = dcp.FileSystemReader(os.path.join(exp, "checkpoint", "step-2")).read_metadata().state_dict_metadata
    keys = set(meta)
    assert not [k for k in keys if "flame_b200" in k], "private keys in the checkpoint"
    assert {"lr_scheduler.last_epoch", "lr_scheduler._step_count", "train_state.step", "dataloader.rank_0"} <= keys
    assert any(k.startswith("optimizer.state.") and k.endswith(".exp_avg") for k in keys)
    assert any(k.startswith("optimizer.param_groups.") and k.endswith(".lr") for k in keys)

    # (1) ours -> reference's DCP-to-HF script -> fla model
    class FakeTokenizer:
        @staticmethod
        def from_pretrained(*a, **k):
            return FakeTokenizer()

        def save_pretrained(self, path):
            pass

    to_hf.AutoTokenizer = FakeTokenizer   # no tokenizer files without a network; everything else is the script's own
    real_auto = to_hf.AutoModelForCausalLM

    class AutoShim:
        """The installed fla declares ``_tied_weights_keys`` as a list, which the installed transformers' ``save_pretrained``
        no longer accepts; the shim hands the script the same fla model with that attribute in the new (mapping) form."""
        @staticmethod
        def from_config(config):
            m = real_auto.from_config(config)
            for sub in m.modules():
                if isinstance(getattr(sub, "_tied_weights_keys", None), list):
                    sub._tied_weights_keys = {}
            return m

    to_hf.AutoModelForCausalLM = AutoShim
    to_hf.save_pretrained(exp, 2, os.path.join(tmp, "tiny.json"), "unused")
    from transformers import AutoModelForCausalLM
    theirs = AutoModelForCausalLM.from_pretrained(exp)
    ours = build_model(ModelConfig.from_pretrained(os.path.join(tmp, "tiny.json")), device="cpu", init=False)
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
    import io
    from datetime import timedelta
    dcp_to_torch_save(os.path.join(exp, "checkpoint", "step-2"), os.path.join(tmp, "flat.pt"))
    torch.serialization.add_safe_globals([timedelta, io.BytesIO])
    flat = torch.load(os.path.join(tmp, "flat.pt"), map_location="cpu", weights_only=False)["model"]
    tsd = theirs.state_dict()
    assert set(tsd) == set(flat), (sorted(set(tsd) ^ set(flat))[:6])
    for k, v in flat.items():
        assert torch.equal(v.to(tsd[k].dtype), tsd[k]), k

    # (2) reference's HF-to-DCP script -> our trainer resumes from it as step-0
    with torch.no_grad():
        for p_ in theirs.parameters():
            p_.mul_(0.5)
    hf2 = os.path.join(tmp, "hf2")
    for sub in theirs.modules():
        if isinstance(getattr(sub, "_tied_weights_keys", None), list):
            sub._tied_weights_keys = {}
    theirs.save_pretrained(hf2)
    exp3 = os.path.join(tmp, "exp3")
    to_dcp.convert_hf_weights(hf2, pathlib.Path(exp3) / "checkpoint" / "step-0")
    a3 = [x if x != exp else exp3 for x in _args(tmp, steps=1, extra=["--checkpoint.enable_checkpoint", "--checkpoint.interval",
                                                                     "100", "--checkpoint.load_step", "0"])]
    cfg3 = JobConfig().parse_args(a3)
    cfg3.training.steps = 0  # build, load, do not train: the engine then holds exactly the loaded weights
    from flame_b200 import train as train_mod
    captured = {}
    orig = train_mod.CheckpointManager.load

    def load_and_capture(self, step=-1):
        r = orig(self, step)
        captured["state"] = self.engine.full_state("master")
        return r

    train_mod.CheckpointManager.load = load_and_capture
    try:
        main(cfg3)
    finally:
        train_mod.CheckpointManager.load = orig
    half = theirs.state_dict()
    for k, v in captured["state"].items():
        assert torch.allclose(v, half[k].float()), k
