"""Job configuration: dotted ``--section.key`` flags, TOML overlay, attribute namespaces.

Same surface as the reference (flame/config_manager.py:67-960): precedence is command line > TOML file >
built-in default; TOML keys without a flag definition are kept (the shipped ``fla.toml`` relies on that for
``training.pin_memory``, ``training.persistent_workers`` and ``checkpoint.interval_type``); ``string_list``
values may be given as comma-separated strings.  Flags are declared in one table instead of a long argparse
script, and "was this flag given on the command line" is answered by scanning ``argv`` rather than by a second
parser.
"""
from __future__ import annotations

import argparse
import sys
from typing import Any, Dict, List, Optional, Sequence

import torch

try:
    import tomllib
except ModuleNotFoundError:  # pragma: no cover
    import tomli as tomllib

TORCH_DTYPE_MAP = {"float16": torch.float16, "float32": torch.float32, "bfloat16": torch.bfloat16}


def string_list(raw: Any) -> List[str]:
    if isinstance(raw, (list, tuple)):
        return [str(x) for x in raw]
    return [s for s in str(raw).split(",") if s != ""]


FLAG = "flag"  # store_true marker

# (section, key, type, default, help[, choices])
_SPEC = [
    ("job", "config_file", str, None, "Job config file (TOML)"),
    ("job", "dump_folder", str, "./torchtitan/outputs", "Folder to dump job outputs"),
    ("job", "description", str, "default job", "Description of the job"),
    ("job", "use_for_integration_test", FLAG, False, "Add this config to the integration test suite"),
    ("job", "print_args", FLAG, False, "Print the args to the terminal"),
    ("model", "name", str, "fla", "Which train spec to use"),
    ("model", "config", str, "fla-hub/transformer-1.3B-100B", "Path to the model config (JSON file or directory)"),
    ("model", "tokenizer_path", str, "fla-hub/transformer-1.3B-100B", "Tokenizer path"),
    ("model", "converters", string_list, [], "Comma separated list of model converters (e.g. float8)"),
    ("model", "print_after_conversion", FLAG, False, "Print the model after converters were applied"),
    ("profiling", "enable_profiling", FLAG, False, "Enable the torch profiler"),
    ("profiling", "save_traces_folder", str, "profile_traces", "Trace files location"),
    ("profiling", "profile_freq", int, 10, "How often to collect profiler traces, in iterations"),
    ("profiling", "enable_memory_snapshot", FLAG, False, "Enable CUDA memory snapshots"),
    ("profiling", "save_memory_snapshot_folder", str, "memory_snapshot", "Memory snapshot files location"),
    ("optimizer", "name", str, "AdamW", "Optimizer to use"),
    ("optimizer", "eps", float, 1e-8, "Epsilon value"),
    ("optimizer", "lr", float, 8e-4, "Learning rate"),
    ("optimizer", "beta1", float, 0.9, "Exponential moving average hyperparameter for the first moment"),
    ("optimizer", "beta2", float, 0.95, "Exponential moving average hyperparameter for the second moment"),
    ("optimizer", "weight_decay", float, 0.1, "Weight decay"),
    ("optimizer", "implementation", str, "fused", "Optimizer implementation", ["for-loop", "foreach", "fused"]),
    ("optimizer", "early_step_in_backward", FLAG, False, "Apply the optimizer step during the backward pass"),
    ("lr_scheduler", "warmup_steps", int, 200, "Steps for lr scheduler warmup"),
    ("lr_scheduler", "decay_ratio", float, None, "Ratio of training steps used for the decay phase (WSD)"),
    ("lr_scheduler", "decay_type", str, "linear", "Learning rate decay type", ["linear", "sqrt", "cosine"]),
    ("lr_scheduler", "lr_min", float, 0.0, "Minimum lr ratio at the end of the decay"),
    ("training", "batch_size", int, 8, "Batch size per data-parallel rank"),
    ("training", "seq_len", int, 2048, "Sequence length"),
    ("training", "context_len", int, 2048, "Max length allowed for each document"),
    ("training", "varlen", FLAG, False, "Pack variable-length documents into one row with cu_seqlens"),
    ("training", "gradient_accumulation_steps", int, 1, "Number of steps to accumulate gradients"),
    ("training", "steps", int, 10000, "How many train steps to run"),
    ("training", "max_norm", float, 1.0, "Max norm for gradient clipping"),
    ("training", "skip_nan_inf", FLAG, False, "Skip the update when the gradient norm is NaN or Inf"),
    ("training", "dataset", str, "HuggingFaceFW/fineweb-edu", "Dataset(s) to use, comma separated"),
    ("training", "dataset_name", str, None, "Dataset config name(s)"),
    ("training", "dataset_split", str, None, "Dataset split(s)"),
    ("training", "data_dir", str, None, "Data dir(s)"),
    ("training", "data_files", str, None, "Data file(s)"),
    ("training", "data_probs", str, None, "Sampling probabilities when mixing datasets"),
    ("training", "streaming", FLAG, False, "Load the dataset in streaming mode"),
    ("training", "num_workers", int, 32, "Data loading workers per rank"),
    ("training", "prefetch_factor", int, 2, "Batches loaded in advance by each worker"),
    ("training", "data_parallel_replicate_degree", int, 1, "Degree of replicated (DDP/HSDP) data parallelism"),
    ("training", "data_parallel_shard_degree", int, -1, "Degree of sharded (FSDP) data parallelism; -1 = the rest"),
    ("training", "enable_cpu_offload", FLAG, False, "Keep the fp32 master weights and the AdamW moments in pinned host memory"),
    ("training", "tensor_parallel_degree", int, 1, "Tensor parallel degree"),
    ("training", "disable_loss_parallel", FLAG, False, "Do not shard the loss computation under tensor parallelism"),
    ("training", "fsdp_reshard_after_forward", str, "default", "FSDP reshard-after-forward policy", ["default", "always", "never"]),
    ("training", "mixed_precision_param", str, "bfloat16", "Compute dtype of the parameters", ["bfloat16", "float32"]),
    ("training", "mixed_precision_reduce", str, "float32", "Gradient reduction dtype", ["float32"]),
    ("training", "compile", FLAG, False, "Accepted for compatibility; kernels here are ahead-of-time compiled"),
    ("training", "gc_freq", int, 50, "Python garbage collection frequency, in steps"),
    ("training", "seed", int, 42, "Random seed"),
    ("training", "deterministic", FLAG, False, "Use deterministic algorithms wherever possible"),
    ("metrics", "log_freq", int, 10, "How often to log metrics, in iterations"),
    ("metrics", "enable_tensorboard", FLAG, False, "Log metrics to TensorBoard"),
    ("metrics", "disable_color_printing", FLAG, False, "Disable color in console logs"),
    ("metrics", "save_tb_folder", str, "tb", "Folder for TensorBoard files"),
    ("metrics", "save_for_all_ranks", FLAG, False, "Write metrics on every rank instead of one"),
    ("metrics", "enable_wandb", FLAG, False, "Log metrics to Weights & Biases"),
    ("experimental", "enable_async_tensor_parallel", FLAG, False, "Overlap tensor-parallel collectives with GEMMs"),
    ("experimental", "pipeline_parallel_degree", int, 1, "Pipeline parallel degree"),
    ("experimental", "pipeline_parallel_split_points", string_list, [], "Layer names that begin a new stage"),
    ("experimental", "pipeline_parallel_schedule", str, "1F1B", "Pipeline schedule: GPipe, 1F1B, Interleaved1F1B, LoopedBFS"),
    ("experimental", "pipeline_parallel_schedule_csv", str, "", "Path to a CSV pipeline schedule"),
    ("experimental", "pipeline_parallel_microbatches", int, None, "Number of pipeline microbatches"),
    ("experimental", "enable_compiled_autograd", FLAG, False, "Accepted for compatibility; no effect"),
    ("experimental", "context_parallel_degree", int, 1, "Context parallel degree"),
    ("experimental", "context_parallel_rotate_method", str, "allgather", "How K/V shards move between CP ranks"),
    ("experimental", "custom_model_path", str, "", "Python module path to import for custom model registration"),
    ("checkpoint", "enable_checkpoint", FLAG, False, "Whether to enable checkpointing"),
    ("checkpoint", "folder", str, "checkpoint", "Checkpoint folder under dump_folder"),
    ("checkpoint", "initial_load_path", str, None, "Checkpoint to start from when the folder is empty"),
    ("checkpoint", "initial_load_model_weights_only", FLAG, True, "Load only model weights from initial_load_path"),
    ("checkpoint", "interval", int, 500, "Checkpointing interval in steps"),
    ("checkpoint", "last_save_model_weights_only", FLAG, False, "Save only model weights at the end of training"),
    ("checkpoint", "export_dtype", str, "float32", "dtype of the final model-only export", ["float16", "bfloat16", "float32"]),
    ("checkpoint", "create_seed_checkpoint", FLAG, False, "Initialise the full model and save it as step-0"),
    ("checkpoint", "async_mode", str, "disabled", "disabled | async | async_with_pinned_mem"),
    ("checkpoint", "keep_latest_k", int, 0, "Keep only the latest k checkpoints (0 keeps all)"),
    ("checkpoint", "load_step", int, -1, "Step to load; -1 loads the latest"),
    ("checkpoint", "exclude_from_loading", string_list, [], "Checkpoint keys that are not loaded"),
    ("activation_checkpoint", "mode", str, "selective", "none | selective | full"),
    ("activation_checkpoint", "selective_ac_option", str, "2", "'op', 'mixer' (recompute only the chunk pipelines of linear-attention mixers) or an integer N (checkpoint every Nth block)"),
    ("activation_offload", "mode", str, "none", "none | full: offload saved activations to pinned host memory"),
    ("float8", "enable_fsdp_float8_all_gather", FLAG, False, "All-gather parameters in float8"),
    ("float8", "precompute_float8_dynamic_scale_for_fsdp", FLAG, False, "Precompute float8 scales after each step"),
    ("float8", "force_recompute_fp8_weight_in_bwd", FLAG, False, "Recompute fp8 weights in backward"),
    ("float8", "recipe_name", str, None, "float8 recipe", ["tensorwise", "rowwise", "rowwise_with_gw_hp"]),
    ("comm", "init_timeout_seconds", int, 300, "Timeout of the first collectives"),
    ("comm", "train_timeout_seconds", int, 100, "Timeout after the first train step"),
    ("comm", "trace_buf_size", int, 20000, "Flight recorder ring buffer size (0 disables)"),
    ("memory_estimation", "enabled", FLAG, False, "Estimate memory instead of training"),
    ("memory_estimation", "disable_fake_mode", FLAG, False, "Estimate with real tensors"),
    ("fault_tolerance", "enable", FLAG, False, "Enable replica-level fault tolerance"),
    ("fault_tolerance", "replica_id", int, 0, "Replica id of this group"),
    ("fault_tolerance", "group_size", int, 0, "Number of replica groups"),
    ("fault_tolerance", "min_replica_size", int, 1, "Minimum number of live replicas"),
    ("fault_tolerance", "semi_sync_method", str, None, "Semi-synchronous training over replica groups: local_sgd | diloco"),
    ("fault_tolerance", "sync_steps", int, 5, "Optimizer steps between two synchronisations of the semi-synchronous modes"),
]

NUM_FLAGS = len(_SPEC) + 1  # + the negation flag below


class _Section:
    def __init__(self, **kw: Any) -> None:
        self.__dict__.update(kw)

    def __repr__(self) -> str:
        return f"_Section({self.__dict__})"


class JobConfig:
    """Parse with ``JobConfig().parse_args(argv)``; read as ``cfg.training.seq_len``."""

    def __init__(self) -> None:
        self.args_dict: Dict[str, Dict[str, Any]] = {}
        p = argparse.ArgumentParser(description="flame_b200 trainer", allow_abbrev=False)
        for entry in _SPEC:
            sec, key, typ, default, helptext = entry[:5]
            choices = entry[5] if len(entry) > 5 else None
            name = f"--{sec}.{key}"
            if typ is FLAG:
                if default:
                    p.add_argument(name, action="store_true", default=True, help=helptext)
                else:
                    p.add_argument(name, action="store_true", help=helptext)
            else:
                p.add_argument(name, type=typ, default=default, help=helptext, choices=choices)
        p.add_argument("--checkpoint.no_initial_load_model_weights_only", dest="checkpoint.initial_load_model_weights_only",
                       action="store_false", help="Load the full checkpoint from initial_load_path")
        self.parser = p

    # ------------------------------------------------------------------------------------------------
    def parse_args(self, args_list: Optional[Sequence[str]] = None) -> "JobConfig":
        args_list = list(sys.argv[1:] if args_list is None else args_list)
        args = self.parser.parse_args(args_list)
        flat = vars(args)
        merged: Dict[str, Dict[str, Any]] = {}
        for dotted, v in flat.items():
            sec, key = dotted.split(".", 1)
            merged.setdefault(sec, {})[key] = v
        config_file = merged["job"]["config_file"]
        if config_file:
            with open(config_file, "rb") as f:
                toml_values = tomllib.load(f)
            for sec, kv in toml_values.items():
                merged.setdefault(sec, {}).update(kv)  # unknown keys survive
        # command line wins over TOML: re-apply exactly the flags that were typed
        given = self._given_on_cmdline(args_list)
        for dotted in given:
            sec, key = dotted.split(".", 1)
            merged[sec][key] = flat[dotted]
        # comma-separated strings from TOML for list-typed flags
        for entry in _SPEC:
            sec, key, typ = entry[:3]
            if typ is string_list and isinstance(merged[sec].get(key), str):
                merged[sec][key] = string_list(merged[sec][key])
        self.args_dict = merged
        for sec, kv in merged.items():
            setattr(self, sec, _Section(**kv))
        self._validate()
        return self

    def _given_on_cmdline(self, argv: Sequence[str]) -> List[str]:
        dests = {}
        for action in self.parser._actions:
            for opt in action.option_strings:
                dests[opt] = action.dest
        given = []
        for tok in argv:
            if not tok.startswith("--"):
                continue
            opt = tok.split("=", 1)[0]
            if opt in dests:
                given.append(dests[opt])
        return given

    def _validate(self) -> None:
        assert self.model.config, "--model.config is required"
        assert self.model.tokenizer_path, "--model.tokenizer_path is required"

    def to_dict(self) -> Dict[str, Dict[str, Any]]:
        return self.args_dict
