"""Metrics, logging back ends and device memory statistics.

Reported quantities and their names are those of the reference run logs (torchtitan/components/metrics.py:41-417,
flame/train.py:531-589): ``loss_metrics/global_{avg,max}_loss``, ``throughput(tps)``, ``tflops``, ``mfu(%)``,
``time_metrics/*``, ``memory/*``, ``optimizer/{lr,grad_norm,skipped_step}``.  ``tps`` is tokens per second per
device: ``ntokens / (dt * cp * tp * pp)``; MFU uses the dense bf16 peak of the device (B200: 2.25e15).
"""
from __future__ import annotations

import logging
import os
import time
from datetime import datetime, timedelta
from typing import Any, Dict, Optional

import torch

logger = logging.getLogger("flame_b200")


def init_logger() -> None:
    if logger.handlers:
        return
    logger.setLevel(logging.INFO)
    h = logging.StreamHandler()
    h.setFormatter(logging.Formatter("[flame] %(asctime)s - %(name)s - %(levelname)s - %(message)s"))
    logger.addHandler(h)
    logger.propagate = False


class Color:
    black, red, green, yellow, blue, magenta, cyan, white, reset = (
        "\033[30m", "\033[31m", "\033[32m", "\033[33m", "\033[34m", "\033[35m", "\033[36m", "\033[37m", "\033[39m")


class NoColor:
    black = red = green = yellow = blue = magenta = cyan = white = reset = ""


PEAK_FLOPS = {"B200": 2.25e15, "H200": 989e12, "H100": 989e12, "A100": 312e12}


def get_peak_flops(device_name: str) -> float:
    for k, v in PEAK_FLOPS.items():
        if k in device_name:
            return v
    return 312e12


def get_nparams_and_flops(model, config, seq_len: int):
    """``flops/token = 6 (N - N_embedding) + 12 L H d_head seq_len`` (flame/tools/utils.py:11-41)."""
    nparams = sum(p.numel() for p in model.parameters())
    emb_mod = getattr(model.decoder, "embeddings", None)
    emb = emb_mod.weight.numel() if emb_mod is not None else 0
    heads = config.get("num_heads") or config.get("num_attention_heads") or 1
    l, h = config.num_hidden_layers, heads
    q = config.hidden_size // h
    return nparams, 6 * (nparams - emb) + 12 * l * h * q * seq_len


class DeviceMemoryMonitor:
    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.device_name = torch.cuda.get_device_name(device)
            self.capacity = torch.cuda.get_device_properties(device).total_memory
        else:
            self.device_name, self.capacity = "cpu", 1

    def stats(self) -> Dict[str, float]:
        if not self.cuda:
            return {"max_active_gib": 0.0, "max_active_pct": 0.0, "max_reserved_gib": 0.0, "max_reserved_pct": 0.0,
                    "num_alloc_retries": 0, "num_ooms": 0}
        s = torch.cuda.memory_stats(self.device)
        act, res = s.get("active_bytes.all.peak", 0), s.get("reserved_bytes.all.peak", 0)
        gib = 1024 ** 3
        return {"max_active_gib": act / gib, "max_active_pct": 100 * act / self.capacity,
                "max_reserved_gib": res / gib, "max_reserved_pct": 100 * res / self.capacity,
                "num_alloc_retries": s.get("num_alloc_retries", 0), "num_ooms": s.get("num_ooms", 0)}

    def reset_peak_stats(self) -> None:
        if self.cuda:
            torch.cuda.reset_peak_memory_stats(self.device)


class _NullLogger:
    def log(self, metrics: Dict[str, Any], step: int) -> None:
        pass

    def close(self) -> None:
        pass


class TensorBoardLogger(_NullLogger):
    def __init__(self, log_dir: str) -> None:
        from torch.utils.tensorboard import SummaryWriter
        self.writer = SummaryWriter(log_dir, max_queue=1000)

    def log(self, metrics, step):
        for k, v in metrics.items():
            self.writer.add_scalar(k, v, step)

    def close(self):
        self.writer.close()


class WandBLogger(_NullLogger):
    def __init__(self, log_dir: str, config: Optional[dict] = None) -> None:
        import wandb
        self.wandb = wandb
        wandb.init(project=os.getenv("WANDB_PROJECT", "flame_b200"), dir=log_dir, config=config,
                   id=os.getenv("WANDB_RUN_ID"), name=os.getenv("WANDB_NAME"), resume=os.getenv("WANDB_RESUME", "allow"))

    def log(self, metrics, step):
        self.wandb.log(metrics, step=step)

    def close(self):
        self.wandb.finish()


def build_metric_logger(job_config, rank: int, world_size: int, log_rank: int = 0):
    m = job_config.metrics
    if not (m.save_for_all_ranks or rank == log_rank):
        return _NullLogger()
    dump = job_config.job.dump_folder
    if m.enable_wandb and os.getenv("WANDB_MODE", "") != "disabled":
        try:
            return WandBLogger(dump, job_config.to_dict())
        except Exception as e:
            logger.warning(f"wandb logging unavailable ({e}); continuing without it")
    if m.enable_tensorboard:
        d = os.path.join(dump, m.save_tb_folder, datetime.now().strftime("%Y%m%d-%H%M"))
        if m.save_for_all_ranks:
            d = os.path.join(d, f"rank_{rank}")
        return TensorBoardLogger(d)
    return _NullLogger()


class MetricsProcessor:
    def __init__(self, job_config, dims, device: torch.device, rank: int, world_size: int) -> None:
        self.job_config, self.dims, self.device = job_config, dims, device
        self.logger = build_metric_logger(job_config, rank, world_size, _log_rank(dims, rank, world_size))
        self.monitor = DeviceMemoryMonitor(device)
        self.gpu_peak_flops = get_peak_flops(self.monitor.device_name)
        self.color = NoColor if job_config.metrics.disable_color_printing else Color
        self.ntokens_since_last_log = 0
        self.data_loading_times = []
        self.time_last_log = time.perf_counter()
        self.num_flops_per_token = -1
        self.monitor.reset_peak_stats()

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.job_config.metrics.log_freq == 0

    def log(self, step: int, global_avg_loss: float, global_max_loss: float, extra_metrics: Optional[dict] = None) -> dict:
        dt = time.perf_counter() - self.time_last_log
        tps = self.ntokens_since_last_log / (dt * self.dims.non_data_parallel_size)
        tflops = self.num_flops_per_token * tps / 1e12
        mfu = 100 * self.num_flops_per_token * tps / self.gpu_peak_flops
        e2e = dt / max(self.job_config.metrics.log_freq, 1)
        dl = sum(self.data_loading_times) / max(len(self.data_loading_times), 1)
        mem = self.monitor.stats()
        metrics = {
            "loss_metrics/global_avg_loss": global_avg_loss, "loss_metrics/global_max_loss": global_max_loss,
            "throughput(tps)": tps, "tflops": tflops, "mfu(%)": mfu, "time_metrics/end_to_end(s)": e2e,
            "time_metrics/data_loading(s)": dl, "time_metrics/data_loading(%)": 100 * dl / max(e2e, 1e-9),
            "memory/max_active(GiB)": mem["max_active_gib"], "memory/max_active(%)": mem["max_active_pct"],
            "memory/max_reserved(GiB)": mem["max_reserved_gib"], "memory/max_reserved(%)": mem["max_reserved_pct"],
            "memory/num_alloc_retries": mem["num_alloc_retries"], "memory/num_ooms": mem["num_ooms"],
        }
        if extra_metrics:
            metrics.update(extra_metrics)
        self.logger.log(metrics, step)
        c = self.color
        logger.info(f"{c.red}step: {step:2}  {c.green}loss: {global_avg_loss:7.4f}  "
                    f"{c.yellow}memory: {mem['max_reserved_gib']:5.2f}GiB({mem['max_reserved_pct']:.2f}%)  "
                    f"{c.blue}tps: {round(tps):,}  {c.cyan}tflops: {tflops:,.2f}  {c.magenta}mfu: {mfu:.2f}%{c.reset}")
        self.ntokens_since_last_log = 0
        self.data_loading_times.clear()
        self.time_last_log = time.perf_counter()
        self.monitor.reset_peak_stats()
        return metrics

    def close(self) -> None:
        self.logger.close()


def _log_rank(dims, rank: int, world_size: int) -> int:
    """Metrics come from the first rank of the last pipeline stage (it is the one that sees the loss)."""
    if dims.pp_enabled:
        return (dims.pp - 1) * (world_size // dims.pp)
    return 0
