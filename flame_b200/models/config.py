"""Model configurations.

A model is described by the same HF-style JSON the reference uses (``configs/*.json``, keyed by ``model_type``).
``ModelConfig`` is a plain attribute bag: per-family defaults (the defaults of the corresponding
``fla.models.*Config`` classes) overlaid with the JSON's keys; unknown keys are kept so a config written by
``save_pretrained`` round-trips.  No dependency on ``transformers``.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Any, Dict

_COMMON = dict(
    vocab_size=32000, hidden_size=2048, num_hidden_layers=24, hidden_ratio=4, intermediate_size=None,
    hidden_act="swish", initializer_range=0.02, norm_eps=1e-6, elementwise_affine=True, use_cache=True,
    fuse_norm=True, fuse_swiglu=True, fuse_cross_entropy=True, fuse_linear_cross_entropy=False, use_l2warp=False,
    tie_word_embeddings=False, bos_token_id=1, eos_token_id=2, pad_token_id=None, max_position_embeddings=2048,
    attn=None, attnres_block_size=None,
)

_DEFAULTS: Dict[str, Dict[str, Any]] = {
    "transformer": dict(num_heads=32, num_kv_heads=None, qkv_bias=False, qk_norm=False, window_size=None,
                        rope_theta=10000.0),
    "sba": dict(hidden_size=2048, num_heads=32, num_kv_heads=None, qkv_bias=False, qk_norm=False, window_size=None,
                rope_theta=10000.0, initializer_range=0.006),
    "gla": dict(expand_k=0.5, expand_v=1.0, num_heads=4, num_kv_heads=None, feature_map=None, attn_mode="chunk",
                use_short_conv=False, conv_size=4, use_output_gate=True, clamp_min=None, use_gk=True, use_gv=False,
                gate_logit_normalizer=16, gate_low_rank_dim=16),
    "delta_net": dict(attn_mode="chunk", expand_k=1.0, expand_v=1.0, use_gate=False, use_short_conv=True, conv_size=4,
                      use_beta=True, use_output_norm=True, num_heads=16, qk_norm="l2", qk_activation="silu",
                      allow_neg_eigval=False),
    "gated_deltanet": dict(attn_mode="chunk", expand_v=2.0, use_gate=True, use_short_conv=True, conv_size=4,
                           head_dim=256, num_heads=6, num_v_heads=None, num_hidden_layers=21, allow_neg_eigval=False),
    "gsa": dict(gate_logit_normalizer=8, clamp_min=None, clamp_max=None, num_heads=4, num_kv_heads=None, num_slots=64,
                use_short_conv=False, conv_size=4, expand_k=1, expand_v=1, feature_map="swish", use_output_gate=False,
                use_norm=True),
    "hgrn2": dict(attn_mode="chunk", num_heads=16, expand_ratio=128, use_short_conv=False, conv_size=4,
                  use_lower_bound=True),
    "mamba": dict(state_size=16, num_hidden_layers=48, norm_eps=1e-5, conv_kernel=4, expand=2, use_bias=False,
                  use_conv_bias=True, hidden_act="silu", dt_rank="auto", dt_scale=1.0, dt_min=0.001, dt_max=0.1,
                  dt_init_scheme="random", dt_init_floor=1e-4, rescale_prenorm_residual=False, residual_in_fp32=False,
                  pad_token_id=0),
    "mamba2": dict(state_size=128, num_hidden_layers=48, norm_eps=1e-5, conv_kernel=4, conv_init=None, expand=2,
                   A_init_range=(1, 16), use_bias=False, use_conv_bias=True, hidden_act="silu", dt_min=0.001,
                   dt_max=0.1, dt_init_floor=1e-4, rescale_prenorm_residual=True, residual_in_fp32=True, n_groups=1,
                   head_dim=64, num_heads=None, rmsnorm=True, D_has_hdim=False, norm_before_gate=False, chunk_size=256,
                   pad_token_id=0),
    "samba": dict(hidden_size=2304, state_size=16, num_hidden_layers=18, norm_eps=1e-5, conv_kernel=4, expand=2,
                  use_bias=False, use_conv_bias=True, time_step_rank=144, time_step_scale=1.0, time_step_min=0.001,
                  time_step_max=0.1, time_step_init_scheme="random", time_step_floor=1e-4,
                  attn=dict(layers=[1, 3, 5, 7, 9, 11, 13, 15, 17], num_heads=18, num_kv_heads=18, qkv_bias=False,
                            window_size=2048, rope_theta=10000.0),
                  rescale_prenorm_residual=False, residual_in_fp32=False, pad_token_id=0),
}

#: ``base_model_prefix`` of every family: the attribute under which the decoder stack lives.
BASE_PREFIX = {"mamba": "backbone", "mamba2": "backbone", "samba": "backbone"}


class ModelConfig:
    def __init__(self, model_type: str = "transformer", **kwargs: Any) -> None:
        if model_type not in _DEFAULTS:
            raise ValueError(f"unknown model_type {model_type!r}; known: {sorted(_DEFAULTS)}")
        values = copy.deepcopy(_COMMON)
        values.update(copy.deepcopy(_DEFAULTS[model_type]))
        values.update(kwargs)
        values["model_type"] = model_type
        self.__dict__.update(values)

    # ---- derived quantities ------------------------------------------------------------------------
    @property
    def base_model_prefix(self) -> str:
        return BASE_PREFIX.get(self.model_type, "model")

    def mlp_intermediate_size(self, hidden_size: int | None = None) -> int:
        """Width of the SwiGLU MLP: ``intermediate_size`` or 256 * ceil(D * hidden_ratio * 2/3 / 256)
        (fla/modules/mlp.py:45-49).  For Samba the JSON's ``intermediate_size`` is the Mamba inner size, so the
        MLP width always comes from ``hidden_ratio``."""
        d = hidden_size or self.hidden_size
        if self.intermediate_size is not None and self.model_type != "samba":
            return int(self.intermediate_size)
        inter = int(d * self.hidden_ratio * 2 / 3)
        return 256 * ((inter + 256 - 1) // 256)

    def get(self, key: str, default: Any = None) -> Any:
        return self.__dict__.get(key, default)

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for k, v in self.__dict__.items():
            if isinstance(v, tuple):
                v = list(v)
            out[k] = v
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        mt = d.pop("model_type", "transformer")
        return cls(mt, **d)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        """``path`` is a JSON file or a directory holding ``config.json``."""
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def __repr__(self) -> str:
        return f"ModelConfig {self.to_json_string()}"


def mamba_dt_rank(cfg: ModelConfig) -> int:
    if cfg.model_type == "samba":
        return int(cfg.time_step_rank)
    r = cfg.get("dt_rank", "auto")
    return math.ceil(cfg.hidden_size / 16) if r == "auto" else int(r)
