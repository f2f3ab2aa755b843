"""Small trainer utilities: manual garbage collection, determinism, module import by path, profiling contexts.

Counterparts: torchtitan/tools/utils.py:36-63 (GarbageCollection), torchtitan/distributed/utils.py:83-160
(set_determinism), torchtitan/tools/profiling.py:35-145 (profiler and memory snapshots)."""
from __future__ import annotations

import contextlib
import gc
import importlib
import importlib.util
import os
import pickle
import sys
import time
from typing import Optional

import torch

from ..components.metrics import logger


class GarbageCollection:
    """Disables automatic GC and collects generation 1 every ``gc_freq`` steps so ranks do not stall at
    different moments."""

    def __init__(self, gc_freq: int = 1000) -> None:
        assert gc_freq > 0
        self.gc_freq = gc_freq
        gc.disable()
        gc.collect(1)

    def run(self, step_count: int) -> None:
        if step_count > 1 and step_count % self.gc_freq == 0:
            gc.collect(1)


def set_determinism(seed: Optional[int], deterministic: bool, rank_offset: int = 0) -> int:
    if deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    if seed is None:
        seed = int(time.time()) % (2 ** 31)
        if torch.distributed.is_initialized():
            t = torch.tensor([seed], dtype=torch.int64)
            if torch.distributed.get_backend() == "nccl":
                t = t.cuda()
            torch.distributed.broadcast(t, src=0)
            seed = int(t.item())
    torch.manual_seed(seed + rank_offset)
    return seed


def import_module_from_path(path: str) -> None:
    """Import a python module or package by filesystem path (custom model registration hook)."""
    path = os.path.abspath(path)
    name = os.path.basename(path.rstrip("/")).replace(".py", "")
    if os.path.isdir(path):
        spec = importlib.util.spec_from_file_location(name, os.path.join(path, "__init__.py"),
                                                      submodule_search_locations=[path])
    else:
        spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)


@contextlib.contextmanager
def maybe_enable_profiling(job_config, global_step: int = 0, rank: int = 0):
    p = job_config.profiling
    if not p.enable_profiling:
        yield None
        return
    trace_dir = os.path.join(job_config.job.dump_folder, p.save_traces_folder)
    freq = p.profile_freq
    warmup, active = 3, 1
    wait = max(freq - (active + warmup), 0)

    def handler(prof):
        d = os.path.join(trace_dir, f"iteration_{prof.step_num}")
        os.makedirs(d, exist_ok=True)
        prof.export_chrome_trace(os.path.join(d, f"rank{rank}_trace.json"))

    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts, schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active),
                                on_trace_ready=handler, record_shapes=True) as prof:
        prof.step_num = global_step
        yield prof


@contextlib.contextmanager
def maybe_enable_memory_snapshot(job_config, global_step: int = 0, rank: int = 0):
    p = job_config.profiling
    if not p.enable_memory_snapshot or not torch.cuda.is_available():
        yield None
        return
    folder = os.path.join(job_config.job.dump_folder, p.save_memory_snapshot_folder)
    os.makedirs(folder, exist_ok=True)

    class Snap:
        def __init__(self):
            torch.cuda.memory._record_memory_history(max_entries=100000)
            self.step_num = global_step

        def step(self, exit_ctx: bool = False):
            self.step_num += 1
            if not exit_ctx and self.step_num % p.profile_freq != 0:
                return
            d = os.path.join(folder, f"iteration_{self.step_num}" + ("_exit" if exit_ctx else ""))
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, f"rank{rank}_memory_snapshot.pickle"), "wb") as f:
                pickle.dump(torch.cuda.memory._snapshot(), f)

    s = Snap()
    try:
        yield s
    except torch.OutOfMemoryError:
        s.step(exit_ctx=True)
        raise
