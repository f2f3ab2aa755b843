"""Registration with ``transformers``' Auto classes, so that a directory written by ``CausalLM.save_pretrained`` (or by
``flame_b200.utils.convert_dcp_to_hf``) loads with ``AutoConfig`` / ``AutoModelForCausalLM`` like any other model.

The reference does this for its custom model with three ``register`` calls at import time
(custom_models/sba/__init__.py:1-9, reached through ``--experimental.custom_model_path``, flame/train.py:66-67) and gets
it for free from ``fla`` for the other families.  ``register()`` adds, for every model type of this package that the Auto
classes do not know yet (``sba`` on a machine with ``fla``; all ten without it), a ``PretrainedConfig`` and a
``PreTrainedModel`` whose sub-module names - and therefore state-dict keys - are exactly those of ``CausalLM``.
``override=True`` replaces existing registrations, which routes every family through this package's kernels.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

from .config import _DEFAULTS, ModelConfig
from .modeling import ARCHITECTURES, CausalLM

_REGISTERED: Dict[str, type] = {}


def _make_classes(model_type: str):
    from transformers import PretrainedConfig, PreTrainedModel
    from transformers.modeling_outputs import CausalLMOutputWithPast

    class Config(PretrainedConfig):
        keys_to_ignore_at_inference = ["past_key_values"]

        def __init__(self, **kwargs):
            merged = ModelConfig(model_type, **{k: v for k, v in kwargs.items() if k != "model_type"}).to_dict()
            special = {k: merged.pop(k) for k in ("bos_token_id", "eos_token_id", "pad_token_id", "tie_word_embeddings")
                       if k in merged}
            merged.pop("model_type", None)
            merged.pop("architectures", None)
            for k, v in merged.items():
                setattr(self, k, v)
            super().__init__(**special, **{k: v for k, v in kwargs.items() if k in ("architectures", "torch_dtype", "dtype")})

    Config.model_type = model_type
    Config.__name__ = Config.__qualname__ = f"FlameB200{model_type.title().replace('_', '')}Config"

    class Model(PreTrainedModel):
        config_class = Config
        supports_gradient_checkpointing = False
        _no_split_modules: List[str] = []
        _tied_weights_keys = {}

        def __init__(self, config):
            super().__init__(config)
            d = {k: v for k, v in config.to_dict().items() if not k.startswith("_")}
            d["model_type"] = model_type
            cfg = ModelConfig.from_dict(d) if hasattr(ModelConfig, "from_dict") else ModelConfig(model_type, **{
                k: v for k, v in d.items() if k != "model_type"})
            inner = CausalLM(cfg)
            object.__setattr__(self, "_inner", inner)  # not a registered sub-module: its children are adopted below
            setattr(self, inner.base_model_prefix, inner.decoder)
            self.lm_head = inner.lm_head
            self.post_init()

        def _init_weights(self, module):  # weights come from the checkpoint or from ``CausalLM.init_weights``
            return

        def get_input_embeddings(self):
            return self._inner.decoder.embeddings

        def get_output_embeddings(self):
            return self.lm_head

        def forward(self, input_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                    cu_seqlens: Optional[torch.Tensor] = None, attention_mask=None, **kwargs):
            out = self._inner(input_ids=input_ids, labels=labels, cu_seqlens=cu_seqlens,
                              return_logits=True if labels is not None else None)
            return CausalLMOutputWithPast(loss=out.loss, logits=out.logits)

    Model.base_model_prefix = "backbone" if model_type in ("mamba", "mamba2", "samba") else "model"
    Model.__name__ = Model.__qualname__ = "FlameB200" + ARCHITECTURES.get(model_type, "CausalLM")
    return Config, Model


def register(model_types: Optional[Iterable[str]] = None, override: bool = False) -> List[str]:
    """Registers the given (default: all) model types with ``AutoConfig`` and ``AutoModelForCausalLM``; returns the
    types that were registered by this call."""
    from transformers import AutoConfig, AutoModelForCausalLM
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING
    done = []
    for mt in (list(model_types) if model_types is not None else list(_DEFAULTS)):
        if mt in _REGISTERED:
            continue
        if mt in CONFIG_MAPPING and not override:
            continue
        Config, Model = _make_classes(mt)
        AutoConfig.register(mt, Config, exist_ok=True)
        AutoModelForCausalLM.register(Config, Model, exist_ok=True)
        _REGISTERED[mt] = Model
        done.append(mt)
    return done
