"""Checkpointing in the torch-DCP layout the reference writes and reads.

Layout (flame/train.py:303-327 with the checkpoint manager of its pinned torchtitan, as proven by
flame/utils/convert_dcp_to_hf.py:51 and convert_hf_to_dcp.py:24): ``<dump>/<folder>/step-<N>/`` holding
``.metadata`` + ``__<rank>_<i>.distcp`` with top-level keys

* ``model.<hf fqn>``                               fp32 weights
* ``optimizer.state.<fqn>.{step,exp_avg,exp_avg_sq}`` and ``optimizer.param_groups.<fqn>.<hyper-parameter>``
* ``lr_scheduler.*``, ``dataloader.rank_<k>``, ``train_state.*``

Policy (torchtitan/components/checkpoint.py:447-786): save every ``interval`` steps and at the last step,
``keep_latest_k`` purging, latest step = largest ``step-N`` that has a ``.metadata`` file, a ``step-0`` checkpoint
carries only the model, ``exclude_from_loading``, final model-only export in ``export_dtype``, async modes that
stage to host memory and write from a background thread.

Tensors are handed to DCP as full (unsharded) host tensors, but no rank holds them all: the engine gathers one unit
at a time on the device and only the unit's owner (unit index modulo the shard degree) copies it to the host, so a
rank stages 1/N of the model and of each AdamW moment.  Loading streams one unit at a time.  Any sharding can read
the files - including the reference's FSDP2 DTensors - and the key set is the reference's (no private keys).
"""
from __future__ import annotations

import os
import re
import shutil
import threading
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from .metrics import logger
from .train_state import TrainState

MODEL, OPTIMIZER, LR_SCHEDULER, DATALOADER, TRAIN_STATE = "model", "optimizer", "lr_scheduler", "dataloader", "train_state"


class CheckpointManager:
    def __init__(self, job_config, engine, dataloader, lr_scheduler, train_state: TrainState,
                 rank: int = 0, world_size: int = 1) -> None:
        ck = job_config.checkpoint
        self.cfg = ck
        self.enable = ck.enable_checkpoint
        self.engine, self.dataloader, self.lr_scheduler, self.train_state = engine, dataloader, lr_scheduler, train_state
        self.rank, self.world_size = rank, world_size
        self.folder = os.path.join(job_config.job.dump_folder, ck.folder)
        self.interval = ck.interval
        self.keep_latest_k = ck.keep_latest_k
        if 0 < self.keep_latest_k < 2:
            raise ValueError("checkpoint.keep_latest_k must be 0 (keep all) or at least 2")
        self.async_mode = str(ck.async_mode).lower()
        if self.async_mode not in ("disabled", "async", "async_with_pinned_mem"):
            raise ValueError(f"unknown checkpoint.async_mode {ck.async_mode}")
        self.export_dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[ck.export_dtype]
        self.exclude_from_loading = list(ck.exclude_from_loading)
        self.initial_load_path = ck.initial_load_path
        self.initial_load_model_weights_only = ck.initial_load_model_weights_only
        self.last_save_model_weights_only = ck.last_save_model_weights_only
        self.total_steps = job_config.training.steps
        self._writer: Optional[threading.Thread] = None
        self._writer_error: Optional[BaseException] = None
        self._pg = None
        if self.enable and self.async_mode != "disabled" and dist.is_initialized() and world_size > 1:
            # background writes coordinate over their own CPU group so they never touch the training communicator
            self._pg = dist.new_group(backend="gloo")

    # ---- state assembly ----------------------------------------------------------------------------------
    def _model_state(self, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        return self.engine.full_state("master", partition=True, to_host=True, dtype=dtype)

    def _optimizer_state(self) -> Dict[str, Any]:
        """``torch.optim.AdamW`` state in the flattened form the reference's optimizer container writes
        (torchtitan/components/optimizer.py:97-106): per-parameter ``state.<fqn>.*`` and ``param_groups.<fqn>.*``."""
        o = self.engine.optim
        scal = self.engine.optimizer_scalars()
        ea = self.engine.full_state("exp_avg", partition=True, to_host=True)
        es = self.engine.full_state("exp_avg_sq", partition=True, to_host=True)
        out: Dict[str, Any] = {}
        for fqn in ea:
            out[f"state.{fqn}.step"] = torch.tensor(float(scal["step"]))
            out[f"state.{fqn}.exp_avg"] = ea[fqn]
            out[f"state.{fqn}.exp_avg_sq"] = es[fqn]
            for k, v in (("lr", o.lr), ("betas", (o.beta1, o.beta2)), ("eps", o.eps), ("weight_decay", o.weight_decay),
                         ("amsgrad", False), ("maximize", False), ("foreach", None), ("capturable", False),
                         ("differentiable", False), ("fused", True)):
                out[f"param_groups.{fqn}.{k}"] = v
        return out

    def _small_states(self) -> Dict[str, Any]:
        return {
            LR_SCHEDULER: self.lr_scheduler.state_dict(),
            DATALOADER: self.dataloader.state_dict() if self.dataloader is not None else {},
            TRAIN_STATE: self.train_state.state_dict(),
        }

    def _states(self, model_only: bool = False, dtype: Optional[torch.dtype] = None) -> Dict[str, Any]:
        """What this rank hands to DCP.  Every tensor is a full (unsharded) host tensor, but each rank only holds the
        units it owns (``ShardedEngine.owns_unit``): the job as a whole stages one copy of the model and of each AdamW
        moment, 1/N of it per rank, and the files can be read by any sharding - including the reference's FSDP2."""
        if model_only:
            return {MODEL: self._model_state(dtype)}
        self.train_state.skipped_step = self.engine.skipped_steps()
        return {MODEL: self._model_state(), OPTIMIZER: self._optimizer_state(), **self._small_states()}

    # ---- paths -------------------------------------------------------------------------------------------
    def step_dir(self, step: int, folder: Optional[str] = None) -> str:
        return os.path.join(folder or self.folder, f"step-{step}")

    def find_latest_step(self, folder: Optional[str] = None) -> int:
        folder = folder or self.folder
        if not os.path.isdir(folder):
            return -1
        steps = []
        for name in os.listdir(folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if m and os.path.isfile(os.path.join(folder, name, ".metadata")):
                steps.append(int(m.group(1)))
        return max(steps) if steps else -1

    # ---- save --------------------------------------------------------------------------------------------
    def _should_save(self, step: int, force: bool) -> bool:
        if not self.enable:
            return False
        if force:
            return True
        return step % self.interval == 0

    def save(self, step: int, force: bool = False) -> bool:
        if not self._should_save(step, force):
            return False
        t0 = time.monotonic()
        self.wait()
        last = force and step >= self.total_steps
        model_only = last and self.last_save_model_weights_only
        states = self._states(model_only, self.export_dtype if model_only else None)
        path = self.step_dir(step)
        if self.async_mode == "disabled":
            self._write(states, path)
            self._purge()
        else:
            # the host copies made by _states() are the staging buffers; the write happens off the training thread
            self._writer_error = None

            def work():
                try:
                    self._write(states, path, self._pg)
                    self._purge()
                except BaseException as e:  # surfaced by wait()
                    self._writer_error = e

            self._writer = threading.Thread(target=work, name="ckpt-writer", daemon=True)
            self._writer.start()
        if self.rank == 0:
            logger.info(f"checkpoint step-{step} {'queued' if self.async_mode != 'disabled' else 'saved'} in "
                        f"{time.monotonic() - t0:.2f}s -> {path}")
        return True

    def _write(self, states: Dict[str, Any], path: str, pg=None) -> None:
        os.makedirs(path, exist_ok=True) if self.rank == 0 else None
        if dist.is_initialized() and self.world_size > 1:
            dcp.save(states, checkpoint_id=path, process_group=pg)
        else:
            dcp.save(states, checkpoint_id=path, no_dist=True)

    def maybe_wait_for_staging(self) -> None:
        """Host staging (this rank's 1/N of the state) is done inside ``save``; only the file write is deferred."""
        return

    def wait(self) -> None:
        if self._writer is not None:
            self._writer.join()
            self._writer = None
            if self._writer_error is not None:
                err, self._writer_error = self._writer_error, None
                raise RuntimeError("background checkpoint write failed") from err

    def _purge(self) -> None:
        if self.keep_latest_k <= 0 or self.rank != 0:
            return
        steps = sorted(int(m.group(1)) for m in (re.fullmatch(r"step-(\d+)", n) for n in os.listdir(self.folder)) if m)
        for s in steps[:-self.keep_latest_k]:
            shutil.rmtree(self.step_dir(s), ignore_errors=True)

    # ---- load --------------------------------------------------------------------------------------------
    def load(self, step: int = -1) -> bool:
        """Returns True when a checkpoint was loaded.  Order of preference: ``<folder>/step-<step>`` (or the
        latest), else ``initial_load_path`` (model weights only unless configured otherwise)."""
        if not self.enable and not self.initial_load_path:
            return False
        folder = self.folder
        model_only = False
        if step == -1:
            step = self.find_latest_step()
        if step == -1 or not os.path.isfile(os.path.join(self.step_dir(step), ".metadata")):
            if not self.initial_load_path:
                return False
            path = self.initial_load_path
            if not os.path.isfile(os.path.join(path, ".metadata")):
                s = self.find_latest_step(path)
                if s == -1:
                    raise FileNotFoundError(f"no checkpoint under initial_load_path {path}")
                path = self.step_dir(s, path)
            model_only = self.initial_load_model_weights_only
        else:
            path = self.step_dir(step, folder)
            model_only = step == 0
        t0 = time.monotonic()
        loaded = self._load_from(path, model_only)
        if self.rank == 0:
            logger.info(f"loaded checkpoint {path} in {time.monotonic() - t0:.2f}s (keys: {sorted(loaded)})")
        return True

    def _dcp_load(self, template: Dict[str, Any], path: str) -> None:
        if dist.is_initialized() and self.world_size > 1:
            dcp.load(template, checkpoint_id=path)
        else:
            dcp.load(template, checkpoint_id=path, no_dist=True)

    def _load_from(self, path: str, model_only: bool) -> List[str]:
        """Tensors are read one engine unit at a time (every rank reads the unit's full tensors, keeps its slice and
        drops the rest), so the host never holds more than one unit; the template asks only for the keys that are
        needed, so a checkpoint written by the reference (FSDP2 DTensors, its own optimizer hyper-parameter keys) loads
        too."""
        eng = self.engine
        want = [MODEL] if model_only else [MODEL, OPTIMIZER, LR_SCHEDULER, DATALOADER, TRAIN_STATE]
        want = [k for k in want if k not in self.exclude_from_loading]
        have = set(dcp.FileSystemReader(path).read_metadata().state_dict_metadata.keys())
        step_val = None
        for u in eng.units:
            shapes = {s.fqn: eng.full_shape(s) for s in u.slots}
            if MODEL in want:
                t = {MODEL: {f: torch.empty(shp, dtype=torch.float32) for f, shp in shapes.items()}}
                self._dcp_load(t, path)
                eng.load_full_state(t[MODEL], "master", units=[u])
            if OPTIMIZER in want:
                t = {OPTIMIZER: {}}
                for f, shp in shapes.items():
                    t[OPTIMIZER][f"state.{f}.exp_avg"] = torch.empty(shp, dtype=torch.float32)
                    t[OPTIMIZER][f"state.{f}.exp_avg_sq"] = torch.empty(shp, dtype=torch.float32)
                first = next(iter(shapes))
                if step_val is None:
                    t[OPTIMIZER][f"state.{first}.step"] = torch.zeros(())
                self._dcp_load(t, path)
                opt = t[OPTIMIZER]
                eng.load_full_state({f: opt[f"state.{f}.exp_avg"] for f in shapes}, "exp_avg", units=[u])
                eng.load_full_state({f: opt[f"state.{f}.exp_avg_sq"] for f in shapes}, "exp_avg_sq", units=[u])
                if step_val is None:
                    step_val = float(opt[f"state.{first}.step"])
        small = {k: v for k, v in self._small_states().items() if k in want}
        if DATALOADER in small:
            # only this rank's entry, and only if the checkpoint has it (another data-parallel degree wrote other keys)
            small[DATALOADER] = {k: v for k, v in small[DATALOADER].items() if f"{DATALOADER}.{k}" in have}
            if not small[DATALOADER]:
                small.pop(DATALOADER)
        if LR_SCHEDULER in small:
            small[LR_SCHEDULER] = {k: v for k, v in small[LR_SCHEDULER].items() if f"{LR_SCHEDULER}.{k}" in have}
        if small:
            self._dcp_load(small, path)
        if LR_SCHEDULER in small:
            self.lr_scheduler.load_state_dict(small[LR_SCHEDULER])
        if DATALOADER in small and self.dataloader is not None:
            self.dataloader.load_state_dict(small[DATALOADER])
        if TRAIN_STATE in small:
            self.train_state.load_state_dict(small[TRAIN_STATE])
        if OPTIMIZER in want:
            eng.load_optimizer_scalars({"step": step_val or 0.0, "skipped": float(self.train_state.skipped_step)})
        return want

    def close(self) -> None:
        self.wait()
