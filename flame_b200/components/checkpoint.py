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

Tensors are handed to DCP as full (unsharded) host tensors: the engine gathers one unit at a time, DCP's planner
de-duplicates them across ranks and spreads the writes, and any sharding can load the result - including the
reference's FSDP2 DTensors.
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
        full = self.engine.full_state("master")
        return {k: (v.to(dtype) if dtype is not None else v).cpu() for k, v in full.items()}

    def _optimizer_state(self) -> Dict[str, Any]:
        o = self.engine.optim
        scal = self.engine.optimizer_scalars()
        ea, es = self.engine.full_state("exp_avg"), self.engine.full_state("exp_avg_sq")
        out: Dict[str, Any] = {}
        for fqn in ea:
            out[f"state.{fqn}.step"] = torch.tensor(float(scal["step"]))
            out[f"state.{fqn}.exp_avg"] = ea[fqn].cpu()
            out[f"state.{fqn}.exp_avg_sq"] = es[fqn].cpu()
            for k, v in (("lr", o.lr), ("betas", (o.beta1, o.beta2)), ("eps", o.eps), ("weight_decay", o.weight_decay),
                         ("amsgrad", False), ("maximize", False), ("foreach", None), ("capturable", False),
                         ("differentiable", False), ("fused", True)):
                out[f"param_groups.{fqn}.{k}"] = v
        out["flame_b200.skipped"] = torch.tensor(float(scal["skipped"]))
        return out

    def _states(self, model_only: bool = False, dtype: Optional[torch.dtype] = None) -> Dict[str, Any]:
        if model_only:
            return {MODEL: self._model_state(dtype)}
        return {
            MODEL: self._model_state(),
            OPTIMIZER: self._optimizer_state(),
            LR_SCHEDULER: self.lr_scheduler.state_dict(),
            DATALOADER: self.dataloader.state_dict() if self.dataloader is not None else {},
            TRAIN_STATE: self.train_state.state_dict(),
        }

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
        """Host staging is synchronous here (the copies are made inside ``save``), so there is nothing to wait for."""
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
        template = self._states(model_only=model_only)
        for k in self.exclude_from_loading:
            template.pop(k, None)
        if dist.is_initialized() and self.world_size > 1:
            dcp.load(template, checkpoint_id=path)
        else:
            dcp.load(template, checkpoint_id=path, no_dist=True)
        self._apply(template)
        if self.rank == 0:
            logger.info(f"loaded checkpoint {path} in {time.monotonic() - t0:.2f}s (keys: {sorted(template)})")
        return True

    def _apply(self, states: Dict[str, Any]) -> None:
        if MODEL in states:
            self.engine.load_full_state(states[MODEL], "master")
        if OPTIMIZER in states:
            opt = states[OPTIMIZER]
            ea = {k[len("state."):-len(".exp_avg")]: v for k, v in opt.items() if k.endswith(".exp_avg")}
            es = {k[len("state."):-len(".exp_avg_sq")]: v for k, v in opt.items() if k.endswith(".exp_avg_sq")}
            self.engine.load_full_state(ea, "exp_avg")
            self.engine.load_full_state(es, "exp_avg_sq")
            steps = [float(v) for k, v in opt.items() if k.endswith(".step")]
            self.engine.load_optimizer_scalars({"step": steps[0] if steps else 0.0,
                                                "skipped": float(opt.get("flame_b200.skipped", 0.0))})
        if LR_SCHEDULER in states:
            self.lr_scheduler.load_state_dict(states[LR_SCHEDULER])
        if DATALOADER in states and self.dataloader is not None:
            self.dataloader.load_state_dict(states[DATALOADER])
        if TRAIN_STATE in states:
            self.train_state.load_state_dict(states[TRAIN_STATE])

    def close(self) -> None:
        self.wait()
