"""Train-spec registry: a name -> builders table, as the reference registers its one spec ``"fla"``
(flame/train.py:45-58 on torchtitan/protocols/train_spec.py:43-80).

A spec bundles what the trainer needs to know about a family of models: how to build the model from a config, how to
lay the parallelism over it, and the builders of the components around it.  ``--model.name`` selects the spec;
``register_train_spec`` lets an extension (for example a module named by ``--experimental.custom_model_path``) add its
own without touching the trainer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional


@dataclass
class TrainSpec:
    name: str
    build_model_fn: Callable
    parallelize_fn: Callable
    build_tokenizer_fn: Callable
    build_dataset_fn: Callable
    build_dataloader_fn: Callable
    build_lr_scheduler_fn: Callable
    build_model_config_fn: Callable
    pipelining_fn: Optional[Callable] = None


_SPECS: Dict[str, TrainSpec] = {}


def register_train_spec(spec: TrainSpec) -> None:
    if spec.name in _SPECS:
        raise ValueError(f"Model {spec.name} is already registered.")
    _SPECS[spec.name] = spec


def get_train_spec(name: str) -> TrainSpec:
    if name not in _SPECS:
        raise ValueError(f"Model {name} is not registered (known: {sorted(_SPECS)}).")
    return _SPECS[name]


def _register_default() -> None:
    from .components.lr_scheduler import LRScheduler
    from .data import build_dataloader, build_dataset, build_tokenizer
    from .models import ModelConfig, build_model
    from .parallel.parallelize import parallelize
    from .parallel.pipeline import split_into_stage
    register_train_spec(TrainSpec(name="fla", build_model_fn=build_model, parallelize_fn=parallelize,
                                  build_tokenizer_fn=build_tokenizer, build_dataset_fn=build_dataset,
                                  build_dataloader_fn=build_dataloader, build_lr_scheduler_fn=LRScheduler,
                                  build_model_config_fn=ModelConfig.from_pretrained, pipelining_fn=split_into_stage))


_register_default()
