"""Training entry point: ``python -m flame_b200.train --job.config_file ... [--section.key value ...]``.

Same loop as the reference trainer (flame/train.py:62-622): build tokenizer / data / model, shard, optionally
resume, then per step: gradient accumulation over micro-batches, gradient clipping, optional NaN/Inf skip,
optimizer + schedule, periodic logging (loss averaged and maximised over the data-parallel ranks), periodic
checkpoints, profiler stepping, and the switch from the long start-up timeout to the short training timeout
after step 1.  Differences that matter on a B200: the clip coefficient and the skip decision never leave the
device, inputs are staged in pinned memory and copied asynchronously, and there is no tracing compiler - every
hot op is an ahead-of-time built kernel.
"""
from __future__ import annotations

import json
import os
import time
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist

from .components.checkpoint import CheckpointManager
from .components.lr_scheduler import LRScheduler
from .components.metrics import Color, MetricsProcessor, NoColor, get_nparams_and_flops, init_logger, logger
from .components.train_state import TrainState
from .config_manager import TORCH_DTYPE_MAP, JobConfig
from .ops.varlen import VarlenMeta
from .parallel.dims import ParallelDims
from .parallel.engine import OptimConfig
from .train_spec import get_train_spec
from .tools import utils
from .utils.nvtx import nvtx_range


def init_distributed(job_config: JobConfig, device_type: str) -> None:
    """NCCL on GPUs, gloo on CPUs; asynchronous error handling and the flight recorder are configured through the
    environment before the first communicator exists (torchtitan/distributed/utils.py:242-286)."""
    if dist.is_initialized():
        return
    if "RANK" not in os.environ:
        return
    os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "3")
    tb = job_config.comm.trace_buf_size
    if tb > 0:
        os.environ.setdefault("TORCH_NCCL_TRACE_BUFFER_SIZE", str(tb))
        os.environ.setdefault("TORCH_NCCL_DUMP_ON_TIMEOUT", "1")
        os.environ.setdefault("TORCH_NCCL_DEBUG_INFO_TEMP_FILE",
                              os.path.join(job_config.job.dump_folder, "comm_trace", "rank_"))
    backend = "nccl" if device_type == "cuda" else "gloo"
    dist.init_process_group(backend, timeout=timedelta(seconds=job_config.comm.init_timeout_seconds))


def apply_model_converters(model: torch.nn.Module, job_config: JobConfig) -> None:
    """``--model.converters`` (torchtitan/protocols/model_converter.py:53-80): only ``float8`` is known, as upstream."""
    for name in job_config.model.converters:
        if name == "float8":
            from .ops.float8 import convert_to_float8
            f8 = job_config.float8
            n = convert_to_float8(model, recipe=f8.recipe_name, min_dim=256)
            logger.info(f"float8 converter: {n} projection weights run as tensor-wise fp8 GEMMs"
                        + (" (fp8 all-gather requested: parameters are published in bf16 over peer memory here, "
                           "the flag has no effect)" if f8.enable_fsdp_float8_all_gather else ""))
        else:
            raise ValueError(f"unknown model converter {name!r}")
    if job_config.model.converters and job_config.model.print_after_conversion:
        logger.info(f"Model after conversion:\n{model}")


# flags that parse for compatibility with the reference's recipes but change nothing here: (section, key, inert value, why)
_INERT_FLAGS = [
    ("training", "compile", False, "there is no tracing compiler on this path; every hot op is an ahead-of-time built kernel"),
    ("experimental", "enable_compiled_autograd", False, "there is no tracing compiler on this path"),
    ("experimental", "enable_async_tensor_parallel", False,
     "tensor-parallel collectives are always fused into their GEMMs (that is what the flag asks for)"),
    ("experimental", "context_parallel_rotate_method", "allgather",
     "context parallelism gathers K/V (or passes the recurrent state) in one step; there is no rotation"),
    ("optimizer", "implementation", "fused", "the optimizer is always one fused kernel per shard"),
    ("float8", "precompute_float8_dynamic_scale_for_fsdp", False, "scales are computed inside the cast kernels"),
    ("float8", "force_recompute_fp8_weight_in_bwd", False, "the transposed fp8 weight is always recomputed in backward"),
]


def warn_inert_flags(job_config: JobConfig) -> None:
    """One warning per flag that was set away from its inert value and does nothing in this framework."""
    for sec, key, inert, why in _INERT_FLAGS:
        val = getattr(getattr(job_config, sec, None), key, inert)
        if val != inert:
            logger.warning(f"--{sec}.{key}={val} has no effect: {why}")


def main(job_config: JobConfig) -> TrainState:
    init_logger()
    logger.info(f"Starting job: {job_config.job.description}")
    warn_inert_flags(job_config)
    if job_config.memory_estimation.enabled:
        # estimate and leave, as the reference's estimation entry point does (flame/config_manager.py:824-835)
        from .tools.estimate_memory import estimate
        rep = estimate(job_config, int(os.environ.get("WORLD_SIZE", 1)))
        logger.info("memory estimation per rank:\n" + json.dumps(rep, indent=2))
        return TrainState()
    if job_config.experimental.custom_model_path:
        utils.import_module_from_path(job_config.experimental.custom_model_path)
    color = NoColor if job_config.metrics.disable_color_printing else Color
    if job_config.job.print_args:
        logger.info(f"{color.green}{json.dumps(job_config.to_dict(), indent=2, sort_keys=True, default=str)}{color.reset}")
    gc_handler = utils.GarbageCollection(gc_freq=job_config.training.gc_freq)

    use_cuda = torch.cuda.is_available()
    device_type = "cuda" if use_cuda else "cpu"
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device(f"cuda:{local_rank}") if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    world_size = int(os.environ.get("WORLD_SIZE", 1))
    init_distributed(job_config, device_type)
    rank = dist.get_rank() if dist.is_initialized() else 0

    tr, ex = job_config.training, job_config.experimental
    dims = ParallelDims(dp_shard=tr.data_parallel_shard_degree, dp_replicate=tr.data_parallel_replicate_degree,
                        cp=ex.context_parallel_degree, tp=tr.tensor_parallel_degree, pp=ex.pipeline_parallel_degree,
                        world_size=world_size, enable_loss_parallel=not tr.disable_loss_parallel)
    dims.build_mesh(rank)
    dp_degree, dp_rank = (dims.dp_degree, dims.dp_rank) if dims.dp_enabled else (1, 0)
    ftc = job_config.fault_tolerance
    data_degree, data_rank = dp_degree, dp_rank
    if ftc.enable:
        # every replica group reads its own slice of the data, fixed by its id whatever the current membership
        data_degree, data_rank = dp_degree * max(1, ftc.group_size), ftc.replica_id * dp_degree + dp_rank
    utils.set_determinism(tr.seed, tr.deterministic)
    spec = get_train_spec(job_config.model.name)   # "fla" unless an extension registered another spec
    build_tokenizer, build_dataset, build_dataloader = spec.build_tokenizer_fn, spec.build_dataset_fn, spec.build_dataloader_fn
    build_model, parallelize = spec.build_model_fn, spec.parallelize_fn

    # ---- model config -----------------------------------------------------------------------------
    model_config = spec.build_model_config_fn(job_config.model.config)
    if dims.tp_enabled and model_config.get("fuse_norm", False):
        logger.warning(f"{color.red}Fused norm+gate is evaluated per tensor-parallel shard; disabling fuse_norm.{color.reset}")
        model_config.fuse_norm = False
    if dims.loss_parallel_enabled and model_config.fuse_linear_cross_entropy:
        logger.warning(f"{color.red}Loss parallel enabled: the head runs vocabulary-sharded.{color.reset}")
    tokenizer = build_tokenizer(job_config.model.tokenizer_path, model_config.vocab_size)
    model_config.vocab_size = max(int(getattr(tokenizer, "vocab_size", 0) or 0), model_config.vocab_size)

    # ---- data ---------------------------------------------------------------------------------------
    dataset = build_dataset(dataset=tr.dataset, dataset_name=tr.dataset_name, dataset_split=tr.dataset_split,
                            data_dir=tr.data_dir, data_files=tr.data_files, data_probs=tr.data_probs,
                            streaming=tr.streaming, dp_degree=dp_degree, num_workers=tr.num_workers, seed=tr.seed)
    dataloader = build_dataloader(dataset=dataset, tokenizer=tokenizer, rank=data_rank, world_size=data_degree,
                                  batch_size=tr.batch_size, seq_len=tr.seq_len, context_len=tr.context_len,
                                  varlen=tr.varlen, num_workers=tr.num_workers if dataset != "synthetic" else 0,
                                  pin_memory=getattr(tr, "pin_memory", False),
                                  persistent_workers=getattr(tr, "persistent_workers", False),
                                  snapshot_every_n_steps=job_config.checkpoint.interval, seed=tr.seed,
                                  vocab_size=model_config.vocab_size, prefetch_factor=tr.prefetch_factor)

    # ---- model + sharding ----------------------------------------------------------------------------
    logger.info(f"Building model from the config\n{color.green}{model_config}{color.reset}")
    param_dtype = TORCH_DTYPE_MAP[tr.mixed_precision_param] if use_cuda else torch.float32
    model = build_model(model_config, device="meta", dtype=param_dtype, init=False)
    nparams, flops_per_token = get_nparams_and_flops(model, model_config, tr.context_len)
    apply_model_converters(model, job_config)
    optim = OptimConfig(lr=job_config.optimizer.lr, beta1=job_config.optimizer.beta1, beta2=job_config.optimizer.beta2,
                        eps=job_config.optimizer.eps, weight_decay=job_config.optimizer.weight_decay,
                        max_norm=tr.max_norm, skip_nan_inf=tr.skip_nan_inf, name=job_config.optimizer.name)
    runner = parallelize(model, model_config, dims, job_config, device, param_dtype, optim)
    engine = runner.engine
    engine.init_weights(tr.seed)
    model.train()
    lr_scheduler = spec.build_lr_scheduler_fn(job_config.optimizer.lr, tr.steps, job_config.lr_scheduler.warmup_steps,
                               job_config.lr_scheduler.decay_ratio, job_config.lr_scheduler.decay_type,
                               job_config.lr_scheduler.lr_min)
    train_state = TrainState()
    checkpoint = CheckpointManager(job_config, engine, dataloader, lr_scheduler, train_state, rank, world_size)
    if job_config.checkpoint.create_seed_checkpoint:
        assert world_size == 1, "create the seed checkpoint with a single process"
        checkpoint.enable = True
        checkpoint.save(0, force=True)
        logger.info("Created seed checkpoint")
        return train_state
    checkpoint.load(step=job_config.checkpoint.load_step)

    ft = None
    if ftc.enable:
        from .components.ft import FTManager, connect
        addr = os.environ.get("FLAME_FT_LIGHTHOUSE")
        if not addr:
            raise ValueError("--fault_tolerance.enable needs FLAME_FT_LIGHTHOUSE=host:port (python -m flame_b200.components.ft)")
        ft = FTManager(connect(addr, ftc.replica_id), ftc.replica_id, ftc.group_size, device,
                       timeout=float(os.environ.get("FLAME_FT_TIMEOUT", job_config.comm.train_timeout_seconds)),
                       local_group=dist.group.WORLD if dist.is_initialized() and world_size > 1 else None,
                       local_rank=rank, heartbeat_store=connect(addr, ftc.replica_id))
        semi_sync = None
        if ftc.semi_sync_method:
            # LocalSGD / DiLoCo: the groups train on their own and meet every sync_steps steps
            from .components.ft import SemiSync
            semi_sync = SemiSync(engine, ftc.semi_sync_method, ftc.sync_steps, ft.allreduce, lambda: ft.errored)
        else:
            engine.replica_reducer = ft.allreduce
            engine.commit_gate = ft.should_commit

    metrics = MetricsProcessor(job_config, dims, device, rank, world_size)
    metrics.num_flops_per_token = flops_per_token
    for s, a, m in zip(train_state.log_steps, train_state.global_avg_losses, train_state.global_max_losses):
        metrics.logger.log({"loss_metrics/global_avg_loss": a, "loss_metrics/global_max_loss": m}, s)

    global_batch = tr.batch_size * dp_degree * tr.gradient_accumulation_steps
    tokens_per_step = global_batch * tr.seq_len
    logger.info(f"{color.red}***** Running training *****{color.reset}")
    logger.info(f"  Training starts at step {train_state.step + 1}; model {nparams:,} parameters; "
                f"global batch {global_batch} x seq_len {tr.seq_len} = {tokens_per_step:,} tokens/step; "
                f"{tr.steps:,} steps, warmup {job_config.lr_scheduler.warmup_steps}; "
                f"parallelism {dims.degrees()}")

    if use_cuda:
        from .ops import _lib as _klib
        # device-side waits on other GPUs' flags: long while peers may still be starting up, short in steady state
        _klib.set_peer_wait_seconds(job_config.comm.init_timeout_seconds)
    data_iterator = iter(dataloader)
    accum = tr.gradient_accumulation_steps
    model.loss_grad_scale = 1.0 / accum
    time_begin = time.perf_counter()
    with utils.maybe_enable_profiling(job_config, train_state.step, rank) as profiler, \
            utils.maybe_enable_memory_snapshot(job_config, train_state.step, rank) as mem_profiler:
        while train_state.step < tr.steps:
            if ft is not None:
                dec = ft.start_step(train_state.step)
                if min(dec["steps"].values()) < dec["max_step"]:
                    # a replica group (re)joined behind the others: everyone takes part in copying the state of the
                    # up-to-date group, and the late one continues from that step
                    if ft.recover(engine.replica_state_tensors()) and dec["heal"]:
                        engine.refresh_compute()
                        for _ in range(dec["max_step"] - train_state.step):
                            lr_scheduler.step()
                        train_state.step = dec["max_step"]
                        logger.info(f"fault tolerance: recovered to step {train_state.step} from replica {dec['src']}")
                        if train_state.step >= tr.steps:
                            break
                voided_before = engine.voided_steps
            engine.check_status()  # one pinned host word, no sync: a wait that ran out in an earlier step raises here
            train_state.step += 1
            gc_handler.run(train_state.step)
            engine.zero_grad()
            losses = []
            for micro in range(accum):
                t_data = time.perf_counter()
                with nvtx_range("data"):
                    batch = next(data_iterator)
                metrics.data_loading_times.append(time.perf_counter() - t_data)
                metrics.ntokens_since_last_log += batch["labels"].numel()
                engine.set_last_microbatch(micro == accum - 1)
                with nvtx_range("forward_backward"):
                    losses.append(runner.forward_backward(batch, 1.0 / accum))
            lr = lr_scheduler.get_last_lr()
            with nvtx_range("optimizer"):
                engine.step(lr)
            if ft is not None and engine.voided_steps != voided_before:
                logger.warning(f"fault tolerance: step {train_state.step} was not committed; asking for a new quorum")
                train_state.step -= 1
                continue
            lr_scheduler.step()
            if ft is not None and semi_sync is not None and semi_sync.after_step():
                logger.info(f"fault tolerance: {ftc.semi_sync_method} synchronisation #{semi_sync.syncs} at step {train_state.step}")
            if metrics.should_log(train_state.step):
                loss = torch.stack([l.detach().float() for l in losses]).sum() if losses[0] is not None else torch.zeros((), device=device)
                avg, mx = runner.reduce_loss(loss)
                train_state.skipped_step = engine.skipped_steps()
                train_state.token += tokens_per_step * (train_state.step - (train_state.log_steps[-1] if train_state.log_steps else 0))
                train_state.elapsed += timedelta(seconds=time.perf_counter() - time_begin)
                time_begin = time.perf_counter()
                train_state.log_steps.append(train_state.step)
                train_state.global_avg_losses.append(avg)
                train_state.global_max_losses.append(mx)
                gnorm = engine.grad_norm()
                metrics.log(train_state.step, avg, mx, extra_metrics={"optimizer/lr": lr, "optimizer/grad_norm": gnorm,
                                                                      "optimizer/skipped_step": train_state.skipped_step})
                eta = train_state.elapsed * (tr.steps - train_state.step) / max(train_state.step, 1)
                spent, left = str(train_state.elapsed).split('.')[0], str(eta).split('.')[0]
                logger.info(f"{color.blue}lr: {lr:.4e} gnorm: {gnorm:5.2f} {color.magenta}[{spent:>8}<{left:>8}]{color.reset}")
            checkpoint.save(train_state.step, force=(train_state.step == tr.steps))
            if profiler is not None:
                profiler.step()
            if mem_profiler is not None:
                mem_profiler.step()
            if train_state.step == 1 and dist.is_initialized():
                _set_pg_timeouts(timedelta(seconds=job_config.comm.train_timeout_seconds), device)
            if train_state.step == 1 and use_cuda:
                _klib.set_peer_wait_seconds(job_config.comm.train_timeout_seconds)
    engine.check_status(sync=use_cuda)
    if ft is not None:
        # replica groups that took part in the same quorums hold the same weights: log a fingerprint to compare
        logger.info(f"fault tolerance: replica {ftc.replica_id} ends at step {train_state.step} with parameter "
                    f"checksum {float(sum(u.master.double().sum() for u in engine.units)):.6f} after "
                    f"{ft.reconfigurations} quorum changes and {engine.voided_steps} voided steps")
        ft.shutdown()
    if rank == 0:
        logger.info("Sleeping 2 seconds for other ranks to complete")
        time.sleep(2)
    checkpoint.close()
    metrics.close()
    logger.info("Training completed")
    return train_state


def _set_pg_timeouts(timeout: timedelta, device: torch.device) -> None:
    """Start-up (first compile / first collectives) gets a long timeout, steady-state a short one."""
    dist.barrier(device_ids=[device.index] if device.type == "cuda" else None)
    if device.type == "cuda":
        torch.cuda.synchronize()
    try:
        from torch.distributed.distributed_c10d import _get_default_group
        groups = [_get_default_group()]
        for g in groups:
            if hasattr(dist.distributed_c10d, "_set_pg_timeout"):
                dist.distributed_c10d._set_pg_timeout(timeout, g)
    except Exception as e:  # older backends (gloo) have no adjustable timeout
        logger.debug(f"could not tighten the process-group timeout: {e}")


def cli(argv: Optional[list] = None) -> None:
    init_logger()
    config = JobConfig().parse_args(argv)
    try:
        main(config)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    cli()
