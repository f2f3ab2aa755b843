"""Applies the requested parallelism to a freshly built (meta-device) model and returns a ``Runner``.

Order, as in the reference (flame/models/parallelize_fla.py:36-108): tensor parallelism -> activation
checkpointing -> data-parallel sharding (FSDP / HSDP / DDP are three settings of one engine); pipeline stages are
cut first when ``pipeline_parallel_degree > 1``.  ``training.compile`` is accepted and ignored: there is no tracing
compiler on this path.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.utils.checkpoint as ckpt

from ..components.metrics import logger
from ..ops.varlen import VarlenMeta
from .dims import ParallelDims
from .engine import OptimConfig, ShardedEngine, TorchCollectives


def apply_activation_checkpointing(model, mode: str, option: str) -> None:
    """``full``: every block is recomputed in backward; ``selective`` with an integer N: every Nth block;
    ``selective`` with ``op``: every block is recomputed but keeps the outputs of its attention and of every other
    matrix product (``ops/sac.py``), the policy of flame/models/parallelize_fla.py:284-331; ``selective`` with ``mixer``:
    only the chunk pipelines of the linear-attention token mixers are recomputed (``ops/chunked.py``)."""
    if mode in (None, "none"):
        return
    if mode not in ("full", "selective"):
        raise ValueError(f"invalid activation_checkpoint.mode {mode!r}")
    every = 1
    op_level = mode == "selective" and option == "op"
    if mode == "selective" and option == "mixer":
        # an option of this framework: blocks are not recomputed, only the chunk pipeline of their token mixer is
        from ..ops.chunked import set_mixer_recompute
        set_mixer_recompute(True)
        logger.info("Applied selective activation checkpointing to the token mixers (chunk pipelines are recomputed)")
        return
    if mode == "selective" and not op_level:
        if not str(option).isdigit() or int(option) <= 0:
            raise ValueError(f"Invalid selective AC option: {option}. Valid options: 'op' or a positive int "
                             "representing layer frequency")
        every = int(option)
    counter = {"n": 0}
    chosen = set()
    for blk in model.decoder.layers:
        if blk is None:
            continue
        counter["n"] += 1
        if every == 1 or counter["n"] % every == 0:
            chosen.add(blk.layer_idx)

    def run(layer, x, meta, residual=None, **kw):
        if op_level:
            from ..ops import sac
            tape = sac.Tape()

            def fn(t, r=None):
                tape.begin_run()
                with sac.use(tape):
                    return layer(t, meta, r, **kw)

            args = (x,) if residual is None else (x, residual)
            return ckpt.checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False)
        if layer.layer_idx in chosen:
            if residual is None:
                return ckpt.checkpoint(lambda t: layer(t, meta, None, **kw), x, use_reentrant=False,
                                       preserve_rng_state=False)
            return ckpt.checkpoint(lambda t, r: layer(t, meta, r, **kw), x, residual, use_reentrant=False,
                                   preserve_rng_state=False)
        return layer(x, meta, residual, **kw)

    model.decoder.activation_checkpoint = run
    logger.info(f"Applied {mode} activation checkpointing to {len(chosen)} blocks"
                + (" (operator level: attention and every other matrix product are kept)" if op_level else ""))


class Runner:
    """Executes one micro-batch (host->device copy, forward, backward) for whatever parallel layout was applied."""

    def __init__(self, model, engine: ShardedEngine, dims: ParallelDims, device: torch.device, job_config=None) -> None:
        self.model, self.engine, self.dims, self.device, self.job_config = model, engine, dims, device, job_config
        self.cp = None
        self.pp = None

    def to_device(self, batch: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, VarlenMeta]:
        ids = batch["input_ids"].to(self.device, non_blocking=True)
        labels = batch["labels"].to(self.device, non_blocking=True)
        cu = batch.get("cu_seqlens")
        total = ids.numel()
        if cu is not None:
            cu = cu.reshape(-1)
            meta = VarlenMeta.from_cu_seqlens(cu, total, self.device)
        else:
            meta = VarlenMeta.dense(ids.shape[0], ids.shape[1], self.device)
        return ids, labels, meta

    def forward_backward(self, batch: Dict[str, torch.Tensor], loss_scale: float = 1.0) -> Optional[torch.Tensor]:
        if self.pp is not None:
            return self.pp.forward_backward(batch, loss_scale)
        ids, labels, meta = self.to_device(batch)
        weight = 1.0
        if self.cp is not None:
            ids, labels, meta = self.cp.shard_batch(ids, labels, meta)
            weight = self.cp.loss_weight  # this rank's share of the valid targets, so the group mean is the token mean
        self.model.loss_grad_scale = loss_scale * weight
        out = self.model(input_ids=ids, labels=labels, meta=meta)
        out.loss.backward()
        return out.loss.detach() * (loss_scale * weight)

    def reduce_loss(self, loss: torch.Tensor) -> Tuple[float, float]:
        """(mean, max) of the step loss over the data-parallel x context-parallel ranks."""
        g = self.dims.group("dp_cp")
        if self.pp is not None:
            loss = self.pp.broadcast_loss(loss)
        if g is None:
            v = float(loss)
            return v, v
        pair = torch.stack([loss.float(), loss.float()])
        avg = pair[0:1].clone()
        mx = pair[1:2].clone()
        dist.all_reduce(avg, op=dist.ReduceOp.SUM, group=g)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=g)
        return float(avg) / dist.get_world_size(g), float(mx)


def parallelize(model, model_config, dims: ParallelDims, job_config, device: torch.device, param_dtype: torch.dtype,
                optim: OptimConfig) -> Runner:
    pp_runner = None
    if dims.pp_enabled:
        from .pipeline import split_into_stage
        split_into_stage(model, model_config, dims, job_config)
    if dims.tp_enabled:
        from .tensor_parallel import apply_tensor_parallel
        apply_tensor_parallel(model, model_config, dims, job_config)
    ac = job_config.activation_checkpoint
    apply_activation_checkpointing(model, ac.mode, ac.selective_ac_option)
    engine = None
    offload = bool(getattr(job_config.training, "enable_cpu_offload", False))
    # fsdp_reshard_after_forward (flame/models/parallelize_fla.py:444-456): "never" keeps the gathered parameters
    # resident (one full bf16 copy per rank, the fastest layout on 180 GB parts); "default" / "always" shard them between
    # uses (parallel/resharding.py), which combines with plain data-parallel sharding only
    policy = str(getattr(job_config.training, "fsdp_reshard_after_forward", "default"))
    reshard = (policy in ("default", "always") and dims.dp_shard_enabled and not dims.tp_enabled and not dims.pp_enabled
               and not dims.dp_replicate_enabled and not offload and os.environ.get("FLAME_B200_RESHARD", "1") != "0")
    if policy in ("default", "always") and dims.dp_shard_enabled and not reshard:
        logger.info("fsdp_reshard_after_forward: parameters stay gathered (tensor / pipeline / replicate parallelism or "
                    "optimizer offload is on, which the sharded-parameter mode does not combine with)")
    make_engine = ShardedEngine
    engine_kw = {}
    if reshard:
        from .resharding import ReshardingEngine
        make_engine = ReshardingEngine
        engine_kw = {"policy": policy,
                     "fuse_gather": os.environ.get("FLAME_B200_FUSED_GATHER", "1") != "0" and
                     "float8" not in list(job_config.model.converters)}
    want_peer = (device.type == "cuda" and dims.dp_shard_enabled and not offload
                 and os.environ.get("FLAME_B200_PEER", "1") != "0")
    if want_peer:
        # peer-memory kernels over NVLink.  There is ONE path: if the symmetric buffers cannot be mapped the job stops
        # with that error; the c10d collectives are chosen only on purpose, with FLAME_B200_PEER=0.
        from .peer import PeerCollectives
        try:
            collectives = PeerCollectives(dims, device)
            engine = make_engine(model, dims, device, param_dtype, optim, collectives=collectives,
                                 allocator=collectives.allocate, **engine_kw)
            collectives.attach(engine)
        except Exception as e:
            raise RuntimeError("the peer-memory collectives could not be set up (symmetric-memory allocation or handle "
                               "exchange failed); set FLAME_B200_PEER=0 to run on the c10d collectives instead") from e
        logger.info("gradient reduce-scatter and parameter publication run on peer-memory kernels")
    if engine is None:
        if reshard:
            from .resharding import TorchReshardCollectives
            engine = make_engine(model, dims, device, param_dtype, optim,
                                 collectives=TorchReshardCollectives(dims.group("dp_shard_cp"), dims.group("dp_replicate")),
                                 **engine_kw)
        else:
            engine = ShardedEngine(model, dims, device, param_dtype, optim, cpu_offload=offload)
        if offload:
            logger.info("optimizer state (fp32 master weights, AdamW moments) is kept in pinned host memory")
    if reshard:
        rep = engine.memory_report()
        logger.info(f"sharded-parameter mode ({policy}): {rep['sharded_bytes'] / 2 ** 20:.1f} MiB of sharded state + "
                    f"{rep['staging_bytes'] / 2 ** 20:.1f} MiB of staging per rank for {int(rep['parameters']):,} parameters")
    engine.install_backward_hooks()
    runner = Runner(model, engine, dims, device, job_config)
    if dims.cp_enabled:
        from .context_parallel import ContextParallel
        runner.cp = ContextParallel(dims, model)
    if dims.pp_enabled:
        from .pipeline import PipelineRunner
        runner.pp = PipelineRunner(model, engine, dims, device, job_config)
    if getattr(job_config.activation_offload, "mode", "none") not in ("none", None):
        from .activation_offload import enable_activation_offload
        enable_activation_offload(runner)
    return runner
