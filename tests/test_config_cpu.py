"""Job configuration, learning-rate schedule and optimizer selection (CPU).
Reference behaviour: flame/config_manager.py:28-42, 55, 878-913; torchtitan/components/lr_scheduler.py:84-190;
torchtitan/components/optimizer.py:292-310."""
import math

import pytest
import torch

from flame_b200.components.lr_scheduler import LRScheduler
from flame_b200.config_manager import JobConfig, string_list


def _toml(tmp_path, text):
    p = tmp_path / "job.toml"
    p.write_text(text)
    return str(p)


BASE = ["--model.config", "configs/transformer_340M.json", "--model.tokenizer_path", "synthetic"]


def test_precedence_cmdline_over_toml_over_default(tmp_path):
    f = _toml(tmp_path, "[training]\nseq_len = 4096\nbatch_size = 3\n[optimizer]\nlr = 1e-3\n")
    cfg = JobConfig().parse_args(BASE + ["--job.config_file", f, "--training.batch_size", "7"])
    assert cfg.training.seq_len == 4096          # TOML over default
    assert cfg.training.batch_size == 7          # command line over TOML
    assert cfg.optimizer.lr == 1e-3
    assert cfg.optimizer.beta2 == 0.95           # default
    # a flag typed with its default value still wins over the TOML
    cfg = JobConfig().parse_args(BASE + ["--job.config_file", f, "--optimizer.lr", "8e-4"])
    assert cfg.optimizer.lr == 8e-4


def test_toml_keys_without_a_flag_survive(tmp_path):
    f = _toml(tmp_path, "[training]\npin_memory = true\npersistent_workers = false\n[checkpoint]\ninterval_type = \"steps\"\n"
                        "[custom]\nanything = 5\n")
    cfg = JobConfig().parse_args(BASE + ["--job.config_file", f])
    assert cfg.training.pin_memory is True and cfg.training.persistent_workers is False
    assert cfg.checkpoint.interval_type == "steps" and cfg.custom.anything == 5


def test_shipped_toml_parses_and_defines_what_the_trainer_reads():
    cfg = JobConfig().parse_args(BASE + ["--job.config_file", "flame_b200/models/fla.toml"])
    for key in ("pin_memory", "persistent_workers", "prefetch_factor", "num_workers", "seq_len", "varlen"):
        assert hasattr(cfg.training, key), key


def test_string_list_and_flags(tmp_path):
    assert string_list("a,b,,c") == ["a", "b", "c"] and string_list(["x", 1]) == ["x", "1"]
    cfg = JobConfig().parse_args(BASE + ["--model.converters", "float8,other", "--training.varlen",
                                         "--checkpoint.exclude_from_loading", "dataloader,lr_scheduler"])
    assert cfg.model.converters == ["float8", "other"] and cfg.training.varlen is True
    assert cfg.checkpoint.exclude_from_loading == ["dataloader", "lr_scheduler"]
    f = _toml(tmp_path, "[model]\nconverters = \"float8\"\n[experimental]\npipeline_parallel_split_points = [\"layers.4\"]\n")
    cfg = JobConfig().parse_args(BASE + ["--job.config_file", f])
    assert cfg.model.converters == ["float8"] and cfg.experimental.pipeline_parallel_split_points == ["layers.4"]


def test_negation_flag_and_choices():
    cfg = JobConfig().parse_args(BASE)
    assert cfg.checkpoint.initial_load_model_weights_only is True
    cfg = JobConfig().parse_args(BASE + ["--checkpoint.no_initial_load_model_weights_only"])
    assert cfg.checkpoint.initial_load_model_weights_only is False
    with pytest.raises(SystemExit):
        JobConfig().parse_args(BASE + ["--optimizer.implementation", "magic"])
    with pytest.raises(SystemExit):
        JobConfig().parse_args(BASE + ["--no.such_flag", "1"])


def test_inert_flags_warn(caplog):
    import logging
    from flame_b200.train import warn_inert_flags
    cfg = JobConfig().parse_args(BASE + ["--training.compile", "--optimizer.implementation", "foreach"])
    with caplog.at_level(logging.WARNING, logger="flame_b200"):
        logging.getLogger("flame_b200").propagate = True
        warn_inert_flags(cfg)
    text = " ".join(r.getMessage() for r in caplog.records)
    assert "--training.compile=True has no effect" in text and "--optimizer.implementation=foreach" in text


# ---------------------------------------------------------------------------------------------------------------
def test_lr_schedule_shapes():
    s = LRScheduler(1.0, training_steps=100, warmup_steps=10, decay_ratio=None, decay_type="linear", lr_min=0.0)
    f = [s.factor(i) for i in range(100)]
    assert f[0] == pytest.approx(1 / 11) and f[9] == pytest.approx(10 / 11)      # linear warmup, never 0
    assert f[10] == 1.0                                                        # stable = 100 + 1 - 10 - 90 = 1 step
    assert f[11] == pytest.approx(1 - 1 / 90) and f[99] == pytest.approx(1 - 89 / 90)
    assert all(a >= b for a, b in zip(f[10:], f[11:]))
    # warmup-stable-decay with a cosine tail down to lr_min
    s = LRScheduler(2.0, 1000, warmup_steps=100, decay_ratio=0.2, decay_type="cosine", lr_min=0.1)
    assert s.decay_steps == 200 and s.stable_steps == 701
    assert s.factor(500) == 1.0 and s.factor(800) == 1.0
    assert s.factor(801) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 1 / 200)))
    assert s.factor(5000) == pytest.approx(0.1)
    s.step()
    s.step()
    assert s.get_last_lr() == pytest.approx(2.0 * 3 / 101)
    # sqrt decay, warmup clipped to the run length, decay clipped to what is left
    s = LRScheduler(1.0, 50, warmup_steps=80, decay_ratio=0.5, decay_type="sqrt")
    assert s.warmup_steps == 50 and s.decay_steps == 0
    s = LRScheduler(1.0, 100, warmup_steps=0, decay_type="sqrt")
    assert s.factor(24) == pytest.approx(1 - math.sqrt(24 / 100))
    with pytest.raises(ValueError):
        LRScheduler(1.0, 10, 0, decay_type="exp").factor(5)


def test_lr_schedule_matches_a_lambda_lr_built_the_reference_way():
    """The same three-phase lambda on a real ``LambdaLR`` gives the same learning rates and the same state-dict keys."""
    base, steps, warm = 3e-4, 60, 7
    mine = LRScheduler(base, steps, warm, decay_ratio=0.5, decay_type="linear", lr_min=0.1)
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=base)
    ref = torch.optim.lr_scheduler.LambdaLR(opt, mine.factor)
    for _ in range(steps):
        assert mine.get_last_lr() == pytest.approx(ref.get_last_lr()[0])
        opt.step()
        ref.step()
        mine.step()
    assert set(mine.state_dict()) == set(ref.state_dict())
    assert mine.state_dict()["last_epoch"] == ref.state_dict()["last_epoch"]
    other = LRScheduler(base, steps, warm, decay_ratio=0.5, decay_type="linear", lr_min=0.1)
    other.load_state_dict(ref.state_dict())
    assert other.get_last_lr() == pytest.approx(mine.get_last_lr())


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["AdamW", "Adam"])
def test_optimizer_name_selects_the_update_rule(name):
    from flame_b200.ops import optim as optim_ops
    from flame_b200.parallel.engine import OptimConfig
    o = OptimConfig(lr=1e-2, weight_decay=0.1, name=name, max_norm=0.0)
    p0, g = torch.randn(64, generator=torch.Generator().manual_seed(0)), torch.randn(64, generator=torch.Generator().manual_seed(1))
    ref_p = torch.nn.Parameter(p0.clone())
    ref = getattr(torch.optim, name)([ref_p], lr=o.lr, betas=(o.beta1, o.beta2), eps=o.eps, weight_decay=o.weight_decay)
    p, m, v = p0.clone(), torch.zeros(64), torch.zeros(64)
    ctrl = torch.zeros(optim_ops.CTRL_SIZE)
    for _ in range(3):
        ref_p.grad = g.clone()
        ref.step()
        ctrl[optim_ops.CTRL_NORM_SQ] = float(g.pow(2).sum())
        optim_ops.adamw_step(p, m, v, g, None, ctrl, o.lr, o.beta1, o.beta2, o.eps, o.kernel_weight_decay, o.max_norm, False)
        optim_ops.adamw_finalize(ctrl, o.max_norm, False)
    assert torch.allclose(p, ref_p.detach(), atol=1e-6)


def test_unknown_optimizer_is_an_error():
    from flame_b200.parallel.engine import OptimConfig
    with pytest.raises(NotImplementedError):
        OptimConfig(name="SGD")


def test_memory_estimation_mode():
    from flame_b200.tools.estimate_memory import estimate, state_bytes
    from flame_b200.models import ModelConfig
    cfg = ModelConfig.from_pretrained("configs/transformer_340M.json")
    one = state_bytes(cfg, 1, "never")
    n = one["parameters"]
    assert abs(n - 373.9e6) < 1e6
    assert one["total_bytes"] >= n * 18 and one["total_bytes"] < n * 18 * 1.01          # bf16 + fp32 grad + 12 optimizer
    eight = state_bytes(cfg, 8, "default")
    assert eight["mode"] == "sharded parameters"
    assert eight["sharded_bytes"] < one["total_bytes"] / 8 * 1.1                         # 1/N plus chunk padding
    assert eight["staging_bytes"] < 0.25 * one["total_bytes"]
    job = JobConfig().parse_args(BASE + ["--training.seq_len", "8192", "--training.batch_size", "1",
                                         "--training.data_parallel_shard_degree", "8", "--memory_estimation.enabled"])
    a = estimate(job, world_size=8)
    job.training.seq_len = 16384
    b = estimate(job, world_size=8)
    assert a["shard_degree"] == 8 and a["state_gib"] == b["state_gib"]
    assert 1.8 < b["activations_gib_estimate"] / a["activations_gib_estimate"] < 2.2     # linear in the tokens
    assert 0.5 < a["activations_gib_estimate"] < 20
