"""Loss-curve parity over N steps: the unmodified reference trainer against this framework's trainer, from identical
weights, on identical batches.

    python baseline/loss_curve_parity.py --steps 200 [--out curves.json]

The model is a cut of the flagship recipe that both arms run in seconds (Transformer, 4 layers, hidden 512, 8 heads,
vocabulary 32000; one packed row of 8192 tokens per step, documents of 64..4096 tokens cut at 2048; AdamW lr 3e-4,
eps 1e-15, weight decay 0.1, 20 warm-up steps, cosine decay to 0.1, clipping at 1.0; bf16 compute, fp32 master weights).

1. ``--arm reference`` (child process): ``flame.train.main`` from ``baseline/_ref`` through ``baseline/ref_compat.py``
   initialises the model its own way; the initial weights are written out in the HF layout (config.json + safetensors)
   just before its optimizer is built, and the per-step loss it logs is recorded.
2. ``--arm ours`` (child process): those weights become a step-0 checkpoint with ``flame_b200.utils.convert_hf_to_dcp``
   and ``flame_b200.train.main`` resumes from it; its synthetic data stream is the generator the reference arm was fed from.
3. The parent compares the two curves and prints one JSON object: both curves, the largest and the mean absolute
   difference, and the differences at every 20th step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)

MODEL = {"model_type": "transformer", "hidden_size": 512, "num_hidden_layers": 4, "num_heads": 8, "vocab_size": 32000,
         "hidden_ratio": 4, "hidden_act": "swish", "max_position_embeddings": 8192, "norm_eps": 1e-6,
         "initializer_range": 0.02, "fuse_cross_entropy": True, "fuse_norm": True, "fuse_swiglu": True,
         "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": 2, "rope_theta": 10000.0}
SEQ_LEN, CONTEXT_LEN, LR, WARMUP = 8192, 2048, 3e-4, 20


def common_flags(work: str, steps: int):
    cfg = os.path.join(work, "model.json")
    if not os.path.exists(cfg):
        with open(cfg, "w") as f:
            json.dump(MODEL, f)
    return ["--model.config", cfg, "--model.tokenizer_path", "synthetic", "--optimizer.name", "AdamW", "--optimizer.eps", "1e-15",
            "--optimizer.lr", str(LR), "--optimizer.weight_decay", "0.1", "--lr_scheduler.warmup_steps", str(WARMUP),
            "--lr_scheduler.lr_min", "0.1", "--lr_scheduler.decay_type", "cosine", "--training.batch_size", "1",
            "--training.seq_len", str(SEQ_LEN), "--training.context_len", str(CONTEXT_LEN), "--training.varlen",
            "--training.gradient_accumulation_steps", "1", "--training.steps", str(steps), "--training.max_norm", "1.0",
            "--training.skip_nan_inf", "--training.dataset", "synthetic", "--training.num_workers", "0",
            "--training.seed", "42", "--metrics.log_freq", "1", "--activation_checkpoint.mode", "none"]


def arm_reference(work: str, steps: int) -> None:
    os.environ.update({"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": os.environ.get("MASTER_PORT", "29581"), "WANDB_MODE": "disabled"})
    import torch
    torch.cuda.set_device(0)
    from baseline import ref_compat
    ref_compat.install()
    import torchtitan.components.metrics as tt_metrics
    import torchtitan.components.optimizer as tt_opt
    losses = []
    make = tt_metrics.build_metrics_processor

    def build_metrics(job_config, parallel_dims, *a, **k):
        mp = make(job_config, parallel_dims, *a, **k)
        inner = mp.log

        def log(step, global_avg_loss, global_max_loss, extra_metrics=None):
            losses.append(float(global_avg_loss))
            return inner(step, global_avg_loss, global_max_loss, extra_metrics)

        mp.log = log
        return mp

    tt_metrics.build_metrics_processor = build_metrics
    build_opt = tt_opt.build_optimizers

    def build_optimizers(model_parts, job_config, ft_manager=None):
        from safetensors.torch import save_file
        sd = {}
        for k, v in model_parts[0].state_dict().items():
            t = v.full_tensor() if hasattr(v, "full_tensor") else v
            sd[k] = t.detach().float().cpu().contiguous()
        os.makedirs(os.path.join(work, "init"), exist_ok=True)
        save_file(sd, os.path.join(work, "init", "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(work, "init", "config.json"), "w") as f:
            json.dump(MODEL, f)
        return build_opt(model_parts, job_config, ft_manager)

    tt_opt.build_optimizers = build_optimizers
    import flame.train as ft
    ft.build_optimizers = build_optimizers
    ft.build_metrics_processor = build_metrics
    import bench
    bench.SEQ_LEN, bench.CONTEXT_LEN = SEQ_LEN, CONTEXT_LEN
    batches = bench.make_batches(steps, 0)

    class Loader:
        def __iter__(self):
            return iter(batches)

        def state_dict(self):
            return {}

        def load_state_dict(self, sd):
            return None

    class Tok:
        vocab_size, bos_token_id, eos_token_id, pad_token_id = 32000, None, 2, None

        @classmethod
        def from_pretrained(cls, *a, **k):
            return cls()

    ft.AutoTokenizer = Tok
    ft.build_dataset = lambda **k: None
    ft.build_dataloader = lambda **k: Loader()
    cfg = ft.JobConfig()
    cfg.parse_args(["--job.config_file", os.path.join(HERE, "reference_recipe.toml"), "--job.dump_folder",
                    os.path.join(work, "ref_dump"), *common_flags(work, steps)])
    cfg.checkpoint.enable_checkpoint = False
    cfg.metrics.enable_wandb = False
    ft.main(cfg)
    with open(os.path.join(work, "reference.json"), "w") as f:
        json.dump(losses, f)


def arm_ours(work: str, steps: int) -> None:
    from flame_b200.config_manager import JobConfig
    from flame_b200.train import main
    from flame_b200.utils.convert_hf_to_dcp import convert_hf_weights
    exp = os.path.join(work, "ours")
    convert_hf_weights(os.path.join(work, "init"), os.path.join(exp, "checkpoint", "step-0"))
    cfg = JobConfig().parse_args(["--job.dump_folder", exp, *common_flags(work, steps), "--checkpoint.enable_checkpoint",
                                  "--checkpoint.load_step", "0", "--checkpoint.interval", "1000000",
                                  "--checkpoint.last_save_model_weights_only", "--metrics.disable_color_printing"])
    state = main(cfg)
    with open(os.path.join(work, "ours.json"), "w") as f:
        json.dump([float(x) for x in state.global_avg_losses], f)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--arm", default=None, choices=[None, "reference", "ours"])
    ap.add_argument("--work", default=None)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    if a.arm == "reference":
        return arm_reference(a.work, a.steps)
    if a.arm == "ours":
        return arm_ours(a.work, a.steps)
    work = a.work or tempfile.mkdtemp(prefix="flame_parity_")
    for arm in ("reference", "ours"):
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--arm", arm, "--work", work, "--steps", str(a.steps)],
                           cwd=ROOT, capture_output=True, text=True)
        if r.returncode != 0:
            print(json.dumps({"parity": "unavailable", "arm": arm, "error": (r.stderr or r.stdout)[-1500:]}))
            return
    ref = json.load(open(os.path.join(work, "reference.json")))
    ours = json.load(open(os.path.join(work, "ours.json")))
    n = min(len(ref), len(ours))
    diffs = [abs(x - y) for x, y in zip(ref[:n], ours[:n])]
    res = {"steps": n, "max_abs_diff": max(diffs), "mean_abs_diff": sum(diffs) / n,
           "first_loss": [ref[0], ours[0]], "last_loss": [ref[n - 1], ours[n - 1]],
           "every_20th": [[i + 1, round(ref[i], 4), round(ours[i], 4)] for i in range(0, n, 20)] + [[n, round(ref[n - 1], 4), round(ours[n - 1], 4)]],
           "reference": ref[:n], "ours": ours[:n]}
    if a.out:
        with open(a.out, "w") as f:
            json.dump(res, f)
    print(json.dumps({k: v for k, v in res.items() if k not in ("reference", "ours")}))


if __name__ == "__main__":
    main()
