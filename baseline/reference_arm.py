"""Reference arm of ``bench.py``: the unmodified reference trainer (``baseline/_ref/flame``) on the benchmark recipe.

Install: ``python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the reference>``
(dependency resolution fails offline because ``flash-linear-attention`` is not in the wheelhouse although it is
installed in the image, hence ``--no-deps``).  The package is written against an older torchtitan than the image
ships; ``baseline/ref_compat.py`` adapts the installed torchtitan to the signatures the reference calls.

What runs and is timed is the reference's own ``flame.train.main``: HF ``AutoModelForCausalLM`` -> fla
``TransformerForCausalLM`` (flash-attn + fla Triton kernels), ``parallelize_fla`` (FSDP2), torch fused AdamW, its
clipping / NaN-skip / logging loop.  Only the data source (synthetic packed rows, same generator as our arm) and
the tokenizer object are supplied from outside, because the GPU box has no network.  Timing marks are taken from
the trainer's per-step garbage-collection callback, so the loop itself is untouched.
"""
from __future__ import annotations

import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")


def run(args, seq_len: int, context_len: int, model_json: str) -> dict:
    if not os.path.isdir(os.path.join(REF, "flame")):
        return {"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}
    if "gated_deltanet" in os.path.basename(model_json):
        # the reference's chunk_gated_delta_rule kernel faulted on B200 ("misaligned address"); it is not run again
        return {"impl": "reference", "unavailable": "fla chunk_gated_delta_rule raised 'Triton Error [CUDA]: misaligned "
                                                   "address' on this GPU at these shapes; not run again"}
    if int(getattr(args, "pp", 1)) > 1:
        # flame/train.py:123-126 raises NotImplementedError as soon as the pipeline degree is above one
        return {"impl": "reference", "unavailable": "the reference trainer refuses pipeline parallelism "
                                                   "(flame/train.py:123-126 raises NotImplementedError)"}
    world = int(os.environ.get("WORLD_SIZE", 1))
    if "RANK" not in os.environ:  # plain `python bench.py --impl reference` on one GPU
        os.environ.update({"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                           "MASTER_PORT": os.environ.get("MASTER_PORT", "29577")})
        world = 1
    rank, local_rank = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    import torch
    torch.cuda.set_device(local_rank)
    from baseline import ref_compat
    ref_compat.install()
    import torchtitan.tools.utils as tt_utils

    K, W = args.steps, args.warmup
    if os.environ.get("FLAME_REF_COMPILE", "0") == "1":
        W = max(W, 20)  # torch.compile keeps recompiling until it has seen a few document counts; none of that is timed
    marks = {}

    class TimedGC(tt_utils.GarbageCollection):
        def run(self, step_count):
            if step_count in (W + 1, W + K + 1):
                torch.cuda.synchronize()
                if torch.distributed.is_initialized() and world > 1:
                    torch.distributed.barrier(device_ids=[local_rank])
                    torch.cuda.synchronize()
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks[step_count] = (ev, time.perf_counter())
            super().run(step_count)

    tt_utils.GarbageCollection = TimedGC
    import flame.train as ft  # the reference trainer, unmodified

    sys.path.insert(0, ROOT)
    import bench
    bench.SEQ_LEN, bench.CONTEXT_LEN = seq_len, context_len
    bsz, varlen = int(getattr(args, "batch_size", 1)), bool(getattr(args, "varlen", True))
    batches = bench.make_batches(W + K + 1, rank // int(getattr(args, 'tp', 1)), batch_size=bsz, varlen=varlen)

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

        def __repr__(self):
            return "SyntheticTokenizer(vocab_size=32000, eos=2)"

    ft.AutoTokenizer = Tok
    ft.build_dataset = lambda **k: None
    ft.build_dataloader = lambda **k: Loader()

    toml = os.path.join(HERE, "reference_recipe.toml")
    import tempfile
    dump = tempfile.mkdtemp(prefix="flame_ref_dump_")
    argv = [
        "--job.config_file", toml, "--job.dump_folder", dump, "--model.config", model_json, "--model.tokenizer_path",
        "synthetic", "--optimizer.name", "AdamW", "--optimizer.eps", "1e-15", "--optimizer.lr", "3e-4",
        "--lr_scheduler.warmup_steps", "1024", "--lr_scheduler.lr_min", "0.1", "--lr_scheduler.decay_type", "cosine",
        "--training.batch_size", str(bsz), "--training.seq_len", str(seq_len), "--training.context_len", str(context_len),
        *(["--training.varlen"] if varlen else []), "--training.gradient_accumulation_steps", "1",
        "--training.steps", str(W + K + 1),
        "--training.max_norm", "1.0", "--training.skip_nan_inf", "--training.dataset", "synthetic",
        "--training.num_workers", "0", "--training.seed", "42", "--metrics.log_freq", "1000000",
        "--activation_checkpoint.mode", getattr(args, "ac", "none"),
    ]
    tp = int(getattr(args, "tp", 1))
    if tp > 1:
        argv += ["--training.tensor_parallel_degree", str(tp)]
    if getattr(args, "ac", "none") == "selective":
        argv += ["--activation_checkpoint.selective_ac_option", str(getattr(args, "ac_option", "2")).replace("mixer", "2")]
    if os.path.basename(model_json).startswith("sba"):
        # the reference's own registration hook for its custom model (flame/train.py:66-67); the model's package sits
        # beside the installed reference, copied unmodified from the reference's source tree
        argv += ["--experimental.custom_model_path", os.path.join(REF, "custom_models", "sba")]
    if os.environ.get("FLAME_REF_COMPILE", "0") == "1":
        argv.append("--training.compile")
        # Inductor builds its C++ wrapper with -fopenmp and the compiler named by CXX, which this image presets to a g++
        # installed without libgomp.spec: the build ends in "cannot read spec file 'libgomp.spec'".  The distribution's
        # own g++ has the file, so Inductor's compiler setting is pointed at it (the reference itself is untouched).
        if os.path.exists("/usr/bin/g++"):
            import torch._inductor.config as inductor_config
            inductor_config.cpp.cxx = (None, "/usr/bin/g++")
            os.environ["CXX"] = "/usr/bin/g++"
    cfg = ft.JobConfig()
    cfg.parse_args(argv)
    cfg.checkpoint.enable_checkpoint = False
    cfg.profiling.enable_profiling = False
    cfg.metrics.enable_wandb = False
    cfg.job.print_args = False
    sampler = bench.ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ft.main(cfg)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else {}
    if (W + 1) not in marks or (W + K + 1) not in marks:
        return {"impl": "reference", "unavailable": "the reference trainer ended before the timed window closed"}
    dev_ms = marks[W + 1][0].elapsed_time(marks[W + K + 1][0])
    wall_ms = (marks[W + K + 1][1] - marks[W + 1][1]) * 1e3
    t = torch.tensor([dev_ms, wall_ms], dtype=torch.float64, device="cuda")
    if torch.distributed.is_initialized() and world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()
    if rank != 0:
        return {}
    tokens = seq_len * bsz * (world // tp) * K
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    return {
        "impl": "reference", "metric": "train tokens/s", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"name": getattr(args, "config", None), "model": os.path.splitext(os.path.basename(model_json))[0],
                   "global_batch": bsz * (world // tp), "seq_len": seq_len, "context_len": context_len,
                   "varlen": varlen,
                   "parallelism": (f"fsdp{world // tp}" + (f"xtp{tp}" if tp > 1 else "")) if world > 1
                   else "single (autocast bf16, no sharding)",
                   "compile": os.environ.get("FLAME_REF_COMPILE", "0") == "1",
                   "note": "reference flame.train.main through baseline/ref_compat.py; synthetic loader injected"},
        "clocks": clocks,
        "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "ms_per_step": wall_ms / K,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
    }
