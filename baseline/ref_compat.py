"""Compatibility layer that lets the unmodified reference trainer (``baseline/_ref/flame``) run on this image.

The reference is written against torchtitan @ 0b44d4c; the image ships a newer torchtitan whose builder signatures
and module layout differ.  ``install()`` adapts the *installed torchtitan* to the call signatures the reference
uses - nothing of the reference, of fla, of torch or of this repository's framework is touched or substituted:

* restores symbols that moved or disappeared (``torchtitan.config_manager``, ``torchtitan.distributed.pipeline``,
  ``FTParallelDims`` / ``init_ft_manager``, ``TrainSpec(cls=, config=)``);
* wraps builders whose arguments changed (``ParallelDims(enable_loss_parallel=)``, ``init_distributed(job_config)``,
  ``build_optimizers(model_parts, job_config, ft_manager)``, ``build_lr_schedulers(optimizers, job_config)``,
  ``build_metrics_processor``/``MetricsProcessor.log``, profiling contexts);
* checkpointing is disabled in the benchmark recipe, so ``CheckpointManager`` is a no-op object;
* provides the empty ``custom_models`` namespace package the trainer imports.

The model, kernels (fla Triton + flash-attn), FSDP2 sharding, optimizer and training loop that get timed are the
reference's own stock code path.
"""
from __future__ import annotations

import contextlib
import os
import sys
import types
from dataclasses import dataclass
from typing import Any, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def install() -> None:
    if getattr(install, "_done", False):
        return
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import torch
    import torchtitan
    import torchtitan.components.checkpoint as tt_ckpt
    import torchtitan.components.ft as tt_ft
    import torchtitan.components.lr_scheduler as tt_lr
    import torchtitan.components.metrics as tt_metrics
    import torchtitan.components.optimizer as tt_opt
    import torchtitan.config as tt_config
    import torchtitan.distributed as tt_dist
    import torchtitan.distributed.parallel_dims as tt_pd
    import torchtitan.distributed.utils as tt_du
    import torchtitan.protocols.model_converter as tt_mc
    import torchtitan.protocols.train_spec as tt_ts
    import torchtitan.tools.profiling as tt_prof
    import torchtitan.tools.utils as tt_utils

    # ---- datasets: a dataclass the reference imports for its streaming shuffle (unused by the benchmark) ----
    import datasets.iterable_dataset as ds_it
    if not hasattr(ds_it, "ShufflingConfig"):
        @dataclass
        class ShufflingConfig:
            generator: Any = None
            _original_seed: Optional[int] = None

        ds_it.ShufflingConfig = ShufflingConfig

    # ---- custom_models namespace ------------------------------------------------------------------------
    if "custom_models" not in sys.modules:
        ns = types.ModuleType("custom_models")
        ns.__path__ = []  # namespace package without content
        sys.modules["custom_models"] = ns

    # ---- torchtitan.config_manager ----------------------------------------------------------------------
    cm = types.ModuleType("torchtitan.config_manager")
    cm.TORCH_DTYPE_MAP = tt_config.TORCH_DTYPE_MAP
    cm.JobConfig = tt_config.JobConfig
    sys.modules["torchtitan.config_manager"] = cm
    torchtitan.config_manager = cm

    # ---- torchtitan.distributed.pipeline ----------------------------------------------------------------
    pipe = types.ModuleType("torchtitan.distributed.pipeline")
    try:
        import torchtitan.distributed.pipeline_parallel as tt_pp
        for name in ("build_pipeline_schedule", "generate_split_points", "stage_ids_this_rank"):
            if hasattr(tt_pp, name):
                setattr(pipe, name, getattr(tt_pp, name))
    except Exception:
        pass
    for name in ("build_pipeline_schedule", "generate_split_points", "stage_ids_this_rank"):
        if not hasattr(pipe, name):
            def _missing(*a, _n=name, **k):
                raise NotImplementedError(f"{_n} is not available in the installed torchtitan")
            setattr(pipe, name, _missing)
    sys.modules["torchtitan.distributed.pipeline"] = pipe
    tt_dist.pipeline = pipe

    # ---- ParallelDims -----------------------------------------------------------------------------------
    Base = tt_pd.ParallelDims

    class ParallelDims(Base):
        def __init__(self, dp_replicate, dp_shard, cp, tp, pp, world_size, enable_loss_parallel=True, ep=1, **kw):
            self.enable_loss_parallel = enable_loss_parallel
            super().__init__(dp_replicate=dp_replicate, dp_shard=dp_shard, cp=cp, tp=tp, pp=pp, ep=ep,
                             world_size=world_size)

        def build_mesh(self, device_type: Optional[str] = None):
            try:
                return super().build_mesh()
            except TypeError:
                return super().build_mesh(device_type)

        @property
        def loss_parallel_enabled(self):
            return self.tp > 1 and self.enable_loss_parallel

    tt_pd.ParallelDims = ParallelDims
    tt_dist.ParallelDims = ParallelDims

    # ---- fault tolerance stubs --------------------------------------------------------------------------
    class _FT:
        enabled = False
        manager = None
        replicate_pg = None

    tt_ft.FTParallelDims = ParallelDims
    tt_ft.init_ft_manager = lambda job_config: _FT()

    # ---- distributed utils --------------------------------------------------------------------------------
    _init_dist = tt_du.init_distributed

    def init_distributed(job_config):
        if torch.distributed.is_initialized():
            return
        comm = types.SimpleNamespace(init_timeout_seconds=job_config.comm.init_timeout_seconds,
                                     train_timeout_seconds=job_config.comm.train_timeout_seconds,
                                     trace_buf_size=0, save_traces_folder="comm_traces")
        try:
            return _init_dist(comm, enable_cpu_backend=False, base_folder=job_config.job.dump_folder)
        except TypeError:
            return _init_dist(comm)

    tt_du.init_distributed = init_distributed

    # ---- TrainSpec ------------------------------------------------------------------------------------------
    @dataclass
    class TrainSpec:
        name: str
        cls: Any = None
        config: Any = None
        parallelize_fn: Any = None
        pipelining_fn: Any = None
        build_optimizers_fn: Any = None
        build_lr_schedulers_fn: Any = None
        build_dataloader_fn: Any = None
        build_tokenizer_fn: Any = None
        build_loss_fn: Any = None

    _specs: dict = {}
    tt_ts.TrainSpec = TrainSpec
    tt_ts.register_train_spec = lambda spec: _specs.__setitem__(spec.name, spec)
    tt_ts.get_train_spec = lambda name: _specs[name]

    # ---- optimizers / schedulers --------------------------------------------------------------------------
    _build_opt = tt_opt.build_optimizers

    def build_optimizers(model_parts, job_config, ft_manager=None):
        oc = job_config.optimizer
        cfg = types.SimpleNamespace(name=oc.name, lr=oc.lr, beta1=oc.beta1, beta2=oc.beta2, eps=oc.eps,
                                    weight_decay=oc.weight_decay, implementation=oc.implementation,
                                    early_step_in_backward=oc.early_step_in_backward)
        pd = types.SimpleNamespace(ep_enabled=False, pp_enabled=False, dp_replicate_enabled=False)
        return _build_opt(model_parts, cfg, pd, None)

    tt_opt.build_optimizers = build_optimizers

    _build_lr = tt_lr.build_lr_schedulers

    def build_lr_schedulers(optimizers, job_config):
        lc = job_config.lr_scheduler
        cfg = types.SimpleNamespace(warmup_steps=lc.warmup_steps, decay_ratio=lc.decay_ratio, decay_type=lc.decay_type,
                                    min_lr_factor=lc.lr_min, lr_min=lc.lr_min)
        return _build_lr(optimizers, cfg, job_config.training.steps)

    tt_lr.build_lr_schedulers = build_lr_schedulers

    # ---- metrics -------------------------------------------------------------------------------------------
    class MetricsProcessor:
        def __init__(self, job_config, parallel_dims):
            import time
            self.job_config, self.parallel_dims = job_config, parallel_dims
            self.ntokens_since_last_log = 0
            self.data_loading_times = []
            self.time_last_log = time.perf_counter()
            self.num_flops_per_token = -1
            self.optimizers = None
            self.lr_schedulers = None
            self._time = time

        def should_log(self, step):
            return step == 1 or step % self.job_config.metrics.log_freq == 0

        def log(self, step, global_avg_loss, global_max_loss, extra_metrics=None):
            dt = self._time.perf_counter() - self.time_last_log
            tps = self.ntokens_since_last_log / max(dt, 1e-9)
            tt_utils.logger.info(f"step: {step:2}  loss: {global_avg_loss:7.4f}  tps: {round(tps):,}")
            self.ntokens_since_last_log = 0
            self.data_loading_times.clear()
            self.time_last_log = self._time.perf_counter()

        def close(self):
            pass

    tt_metrics.build_metrics_processor = lambda job_config, parallel_dims, *a, **k: MetricsProcessor(job_config, parallel_dims)
    tt_metrics.ensure_pp_loss_visible = lambda *a, **k: None

    # ---- checkpointing: disabled in the benchmark recipe -------------------------------------------------
    class CheckpointManager:
        def __init__(self, *a, job_config=None, **k):
            if job_config is not None and job_config.checkpoint.enable_checkpoint:
                raise NotImplementedError("the compatibility layer runs the reference with checkpointing disabled")

        def save(self, *a, **k):
            return None

        def load(self, *a, **k):
            return False

        def maybe_wait_for_staging(self):
            return None

        def close(self):
            return None

    tt_ckpt.CheckpointManager = CheckpointManager

    # ---- model converters / profiling / misc ---------------------------------------------------------------
    class _Converters:
        def convert(self, model):
            return None

        def post_optimizer_hook(self, model_parts):
            return None

    def build_model_converters(job_config, parallel_dims):
        if job_config.model.converters:
            raise NotImplementedError("model converters are not available through the compatibility layer")
        return _Converters()

    tt_mc.build_model_converters = build_model_converters

    @contextlib.contextmanager
    def _no_profiling(job_config, *, global_step=0, **k):
        yield None

    tt_prof.maybe_enable_profiling = _no_profiling
    tt_prof.maybe_enable_memory_snapshot = _no_profiling

    if not hasattr(tt_utils, "import_module_from_path"):
        def import_module_from_path(path):
            """What ``--experimental.custom_model_path`` asks for: import the package directory at ``path`` (its
            ``__init__`` registers the model with transformers' Auto classes)."""
            import importlib.util
            import sys
            path = os.path.abspath(path)
            name = os.path.basename(path.rstrip("/"))
            spec = importlib.util.spec_from_file_location(name, os.path.join(path, "__init__.py"),
                                                          submodule_search_locations=[path])
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            spec.loader.exec_module(mod)
            return mod

        tt_utils.import_module_from_path = import_module_from_path

    _set_pg = tt_du.set_pg_timeouts

    def set_pg_timeouts(timeout, world_mesh):
        try:
            return _set_pg(timeout, world_mesh)
        except Exception:
            return None

    tt_du.set_pg_timeouts = set_pg_timeouts
    install._done = True
