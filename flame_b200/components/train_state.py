"""Trainer counters that travel with a checkpoint.

Field set and encodings follow flame/components/checkpoint.py:16-59: scalars as int32/int64 tensors, the
logged loss histories as ``torch.save`` bytes, ``elapsed`` as a ``timedelta``."""
from __future__ import annotations

from dataclasses import dataclass, field
from datetime import timedelta
from io import BytesIO
from typing import Any, Dict, List

import torch


@dataclass
class TrainState:
    step: int = 0
    skipped_step: int = 0
    token: int = 0
    elapsed: timedelta = timedelta(0)
    global_avg_losses: List[float] = field(default_factory=list)
    global_max_losses: List[float] = field(default_factory=list)
    log_steps: List[int] = field(default_factory=list)

    def state_dict(self) -> Dict[str, Any]:
        def blob(x):
            b = BytesIO()
            torch.save(x, b)
            b.seek(0)
            return b
        return {
            "step": torch.tensor(self.step, dtype=torch.int32),
            "skipped_step": torch.tensor(self.skipped_step, dtype=torch.int32),
            "token": torch.tensor(self.token, dtype=torch.int64),
            "elapsed": self.elapsed,
            "global_avg_losses": blob(self.global_avg_losses),
            "global_max_losses": blob(self.global_max_losses),
            "log_steps": blob(self.log_steps),
        }

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        def unblob(b):
            b.seek(0)
            return torch.load(b, weights_only=False)
        self.step = int(sd["step"])
        self.skipped_step = int(sd.get("skipped_step", 0))
        self.token = int(sd["token"])
        self.elapsed = sd["elapsed"]
        self.global_avg_losses = unblob(sd["global_avg_losses"])
        self.global_max_losses = unblob(sd["global_max_losses"])
        self.log_steps = unblob(sd["log_steps"])
