"""Warmup -> (optional stable) -> decay learning-rate schedule.

Same curve as the reference's dependency (torchtitan/components/lr_scheduler.py:84-190): linear warmup over
``warmup_steps``; decay (linear | sqrt | cosine) down to ``lr_min`` x base lr; with ``decay_ratio`` the decay
occupies that fraction of training and a constant phase fills the gap (``stable = steps + 1 - warmup - decay``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional


class LRScheduler:
    def __init__(self, base_lr: float, training_steps: int, warmup_steps: int = 200, decay_ratio: Optional[float] = None,
                 decay_type: str = "linear", lr_min: float = 0.0) -> None:
        self.base_lr, self.training_steps = base_lr, training_steps
        self.warmup_steps = min(int(warmup_steps), training_steps)
        if decay_ratio is not None:
            decay_steps = round(training_steps * decay_ratio)
            if self.warmup_steps + decay_steps > training_steps:
                decay_steps = training_steps - self.warmup_steps
        else:
            decay_steps = training_steps - self.warmup_steps
        self.decay_steps = decay_steps
        self.stable_steps = training_steps + 1 - self.warmup_steps - decay_steps
        self.decay_type, self.lr_min = decay_type, lr_min
        self.last_epoch = 0

    def factor(self, step: int) -> float:
        w, s, d = self.warmup_steps, self.stable_steps, self.decay_steps
        if step < w:
            return float((step + 1) / (w + 1))
        if step < w + s:
            return 1.0
        progress = min(1.0, float(step + 1 - w - s) / max(d, 1))
        if self.decay_type == "linear":
            f = 1.0 - progress
        elif self.decay_type == "sqrt":
            f = 1.0 - math.sqrt(progress)
        elif self.decay_type == "cosine":
            f = 0.5 * (1.0 + math.cos(math.pi * progress))
        else:
            raise ValueError(self.decay_type)
        return self.lr_min + (1.0 - self.lr_min) * f

    def get_last_lr(self) -> float:
        return self.base_lr * self.factor(self.last_epoch)

    def step(self) -> None:
        self.last_epoch += 1

    def state_dict(self) -> Dict[str, Any]:
        """The key set of ``torch.optim.lr_scheduler.LambdaLR.state_dict()`` with a plain-function lambda, which is what
        the reference's scheduler container checkpoints (torchtitan/components/lr_scheduler.py:84-190)."""
        return {"base_lrs": [self.base_lr], "last_epoch": self.last_epoch, "_step_count": self.last_epoch + 1,
                "_is_initial": False, "_get_lr_called_within_step": False, "_last_lr": [self.get_last_lr()],
                "lr_lambdas": [None]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.last_epoch = int(sd.get("last_epoch", 0))
