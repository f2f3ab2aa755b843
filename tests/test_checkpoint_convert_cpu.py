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
