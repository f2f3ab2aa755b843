"""Causal language models for all supported families.

Structure and state-dict names follow the reference's HF models: ``<prefix>.embeddings``, ``<prefix>.layers.N``,
``<prefix>.norm`` (``norm_f`` for the Mamba family), ``lm_head`` and a ``criterion``; ``<prefix>`` is ``model`` or
``backbone`` (fla/models/transformer/modeling_transformer.py:255-445, fla/models/mamba/modeling_mamba.py:45-179,
fla/models/samba/modeling_samba.py:49-183, custom_models/sba/modeling_sba.py:34-407).

Activations are packed ``[T, D]``; ``forward(input_ids [B, S], labels, cu_seqlens)`` flattens the batch and
builds one ``VarlenMeta`` (rows of a non-varlen batch become documents).  Labels are shifted inside the model.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import cross_entropy as ce_ops
from ..ops.norm import rms_norm
from ..ops.varlen import VarlenMeta
from . import layers as L
from .config import ModelConfig, mamba_dt_rank
from .modules import Embedding, GatedMLP, Linear, RMSNorm, ShortConvolution


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None


def _softmax_attention(cfg: ModelConfig, attn_cfg: Optional[dict] = None) -> nn.Module:
    a = attn_cfg or {}
    return L.Attention(
        hidden_size=cfg.hidden_size,
        num_heads=a.get("num_heads", cfg.get("num_heads")),
        num_kv_heads=a.get("num_kv_heads", cfg.get("num_kv_heads")),
        qkv_bias=a.get("qkv_bias", cfg.get("qkv_bias", False)),
        qk_norm=a.get("qk_norm", cfg.get("qk_norm", False)) if not isinstance(cfg.get("qk_norm"), str) else False,
        window_size=a.get("window_size", cfg.get("window_size")),
        rope_theta=a.get("rope_theta", cfg.get("rope_theta", 10000.0)),
        max_position_embeddings=cfg.max_position_embeddings,
        norm_eps=cfg.norm_eps,
    )


def build_mixer(cfg: ModelConfig, layer_idx: int) -> nn.Module:
    mt = cfg.model_type
    hybrid = cfg.get("attn")
    if hybrid is not None and mt not in ("samba",) and layer_idx in hybrid.get("layers", []):
        return _softmax_attention(cfg, hybrid)  # hybrid layers (fla/models/gla/modeling_gla.py:51-62)
    if mt == "transformer":
        return _softmax_attention(cfg)
    if mt == "sba":
        return L.StickBreakingAttention(cfg.hidden_size, cfg.num_heads, cfg.get("num_kv_heads"), cfg.get("qkv_bias", False))
    if mt == "gla":
        return L.GatedLinearAttention(cfg.hidden_size, cfg.expand_k, cfg.expand_v, cfg.num_heads, cfg.num_kv_heads,
                                      cfg.feature_map, cfg.use_short_conv, cfg.conv_size, cfg.use_output_gate,
                                      cfg.elementwise_affine, cfg.norm_eps, cfg.gate_logit_normalizer,
                                      cfg.gate_low_rank_dim, cfg.clamp_min, cfg.fuse_norm)
    if mt == "delta_net":
        return L.DeltaNet(cfg.hidden_size, cfg.expand_k, cfg.expand_v, cfg.num_heads, cfg.use_beta, cfg.use_gate,
                          cfg.use_short_conv, cfg.conv_size, cfg.qk_activation, cfg.qk_norm, cfg.allow_neg_eigval,
                          cfg.norm_eps)
    if mt == "gated_deltanet":
        return L.GatedDeltaNet(cfg.hidden_size, cfg.expand_v, cfg.head_dim, cfg.num_heads, cfg.num_v_heads,
                               cfg.use_gate, cfg.use_short_conv, cfg.conv_size, cfg.allow_neg_eigval, cfg.norm_eps)
    if mt == "gsa":
        return L.GatedSlotAttention(cfg.hidden_size, cfg.expand_k, cfg.expand_v, cfg.num_heads, cfg.num_kv_heads,
                                    cfg.num_slots, cfg.feature_map, cfg.use_short_conv, cfg.conv_size,
                                    cfg.elementwise_affine, cfg.norm_eps, cfg.gate_logit_normalizer)
    if mt == "hgrn2":
        return L.HGRN2Attention(cfg.hidden_size, cfg.num_heads, cfg.expand_ratio, cfg.use_short_conv, cfg.conv_size,
                                cfg.elementwise_affine, cfg.norm_eps, layer_idx)
    if mt in ("mamba", "samba"):
        inner = int(cfg.get("intermediate_size") or cfg.expand * cfg.hidden_size) if mt == "samba" else int(cfg.expand * cfg.hidden_size)
        return L.Mamba(cfg.hidden_size, cfg.state_size, cfg.conv_kernel, inner, mamba_dt_rank(cfg), cfg.use_bias,
                       cfg.use_conv_bias)
    if mt == "mamba2":
        heads = int(cfg.expand * cfg.hidden_size) // cfg.head_dim
        return L.Mamba2(cfg.hidden_size, heads, cfg.head_dim, cfg.state_size, cfg.expand, cfg.n_groups, cfg.conv_kernel,
                        cfg.use_conv_bias, cfg.use_bias, cfg.rmsnorm, cfg.norm_before_gate, cfg.norm_eps,
                        cfg.chunk_size, tuple(cfg.A_init_range), cfg.dt_min, cfg.dt_max, cfg.dt_init_floor)
    raise ValueError(mt)


class Block(nn.Module):
    """Pre-norm block ``x + mixer(norm(x))`` then ``x + mlp(norm(x))`` with the residual add fused into the second
    norm (fla/models/transformer/modeling_transformer.py:90-169)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.attn_norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        self.attn = build_mixer(cfg, layer_idx)
        self.mlp_norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        self.mlp = GatedMLP(cfg.hidden_size, cfg.mlp_intermediate_size())

    def forward(self, x: torch.Tensor, meta: VarlenMeta, residual: Optional[torch.Tensor] = None, **kw):
        """Takes and returns ``(hidden, residual)``: the sum of the two is the residual stream, and it is formed
        inside the next norm kernel instead of by a separate add."""
        if residual is None:
            residual = x
            h = self.attn_norm(x)
        else:
            h, residual = self.attn_norm(x, residual, True)
        h = self.attn(h, meta, **kw) if kw else self.attn(h, meta)
        h, residual = self.mlp_norm(h, residual, True)
        h = self.mlp(h)
        return h, residual


class MambaBlock(nn.Module):
    """``x + mixer(norm(x))`` (fla/models/mamba/modeling_mamba.py:45-103)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        self.mixer = build_mixer(cfg, layer_idx)

    def forward(self, x: torch.Tensor, meta: VarlenMeta, residual: Optional[torch.Tensor] = None):
        if residual is None:
            residual = x
            h = self.norm(x)
        else:
            h, residual = self.norm(x, residual, True)
        return self.mixer(h, meta), residual


class SambaBlock(nn.Module):
    """Mamba on even layers, windowed softmax attention on the listed layers, each followed by an MLP
    (fla/models/samba/modeling_samba.py:49-118)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.mixer_norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        attn = cfg.get("attn")
        if attn is not None and layer_idx in attn["layers"]:
            self.mixer = _softmax_attention(cfg, attn)
        else:
            self.mixer = build_mixer(cfg, layer_idx)
        self.mlp_norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        self.mlp = GatedMLP(cfg.hidden_size, cfg.mlp_intermediate_size())

    def forward(self, x: torch.Tensor, meta: VarlenMeta, residual: Optional[torch.Tensor] = None):
        if residual is None:
            residual = x
            h = self.mixer_norm(x)
        else:
            h, residual = self.mixer_norm(x, residual, True)
        h = self.mixer(h, meta)
        h, residual = self.mlp_norm(h, residual, True)
        return self.mlp(h), residual


class Decoder(nn.Module):
    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.config = cfg
        self.embeddings = Embedding(cfg.vocab_size, cfg.hidden_size)
        mt = cfg.model_type
        if mt in ("mamba", "mamba2"):
            self.layers = nn.ModuleList([MambaBlock(cfg, i) for i in range(cfg.num_hidden_layers)])
            self.norm_f = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        elif mt == "samba":
            self.layers = nn.ModuleList([SambaBlock(cfg, i) for i in range(cfg.num_hidden_layers)])
            self.norm_f = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        else:
            self.layers = nn.ModuleList([Block(cfg, i) for i in range(cfg.num_hidden_layers)])
            self.norm = RMSNorm(cfg.hidden_size, eps=cfg.norm_eps)
        if mt == "hgrn2" and cfg.use_lower_bound:
            self.lower_bounds = nn.Parameter(torch.zeros(cfg.num_hidden_layers, cfg.hidden_size))
        self.activation_checkpoint: Optional[callable] = None

    @property
    def final_norm(self) -> Optional[RMSNorm]:
        n = getattr(self, "norm", None)
        return n if n is not None else getattr(self, "norm_f", None)

    def forward(self, input_ids: Optional[torch.Tensor], meta: VarlenMeta,
                inputs_embeds: Optional[torch.Tensor] = None,
                stage: Optional[Tuple[int, int, bool, bool]] = None) -> torch.Tensor:
        """``stage = (first layer, end layer, is first stage, is last stage)`` runs one pipeline stage of a rank that
        holds several: only that layer range, the embeddings only on the first stage, the final norm only on the last."""
        lo, hi, is_first, is_last = stage if stage is not None else (0, len(self.layers), True, True)
        if getattr(self, "embeddings", None) is not None and inputs_embeds is None and is_first:
            x = self.embeddings(input_ids.reshape(-1))
        else:
            x = inputs_embeds
        lbs = None
        if hasattr(self, "lower_bounds"):
            lb = self.lower_bounds.float().softmax(0)
            lbs = lb.cumsum(0) - lb[0]
        residual = None
        for idx, layer in enumerate(self.layers):
            if layer is None or not (lo <= idx < hi):
                continue
            kw = {}
            if lbs is not None:
                kw = {"lower_bound": lbs[layer.layer_idx]}
            if self.activation_checkpoint is not None and self.training:
                x, residual = self.activation_checkpoint(layer, x, meta, residual, **kw)
            else:
                x, residual = layer(x, meta, residual, **kw)
        fn = self.final_norm if is_last else None
        if fn is not None:
            x = fn(x, residual) if residual is not None else fn(x)
        elif residual is not None:
            x = x + residual  # a pipeline stage without the final norm hands on the plain residual stream
        return x


class CausalLM(nn.Module):
    """``<prefix>`` decoder + ``lm_head`` + loss.  ``fuse_linear_cross_entropy`` (or ``fuse_cross_entropy`` on a GPU,
    where materialising [T, V] logits is pure overhead) routes the head through the chunked linear+CE op."""

    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.config = cfg
        self.base_model_prefix = cfg.base_model_prefix
        setattr(self, self.base_model_prefix, Decoder(cfg))
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size)
        self.loss_grad_scale = 1.0
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.decoder.embeddings.weight

    # -- structure ---------------------------------------------------------------------------------
    @property
    def decoder(self) -> Decoder:
        return getattr(self, self.base_model_prefix)

    @classmethod
    def from_config(cls, cfg: ModelConfig) -> "CausalLM":
        return cls(cfg)

    # -- forward -----------------------------------------------------------------------------------
    def forward(self, input_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None,
                meta: Optional[VarlenMeta] = None, inputs_embeds: Optional[torch.Tensor] = None,
                return_logits: Optional[bool] = None,
                stage: Optional[Tuple[int, int, bool, bool]] = None) -> CausalLMOutput:
        ref = input_ids if input_ids is not None else inputs_embeds
        dev = ref.device
        if input_ids is not None and getattr(self.decoder, "embeddings", None) is None and inputs_embeds is None:
            raise ValueError("this pipeline stage has no embeddings: pass inputs_embeds")
        if meta is None:
            if cu_seqlens is not None:
                total = ref.shape[0] * ref.shape[1] if input_ids is not None else ref.shape[0]
                meta = VarlenMeta.from_cu_seqlens(cu_seqlens, total, dev)
            else:
                B, S = ref.shape[:2]
                meta = VarlenMeta.dense(B, S, dev)
        hidden = self.decoder(input_ids, meta, inputs_embeds, stage)
        if getattr(self, "lm_head", None) is None or (stage is not None and not stage[3]):
            # a pipeline stage without the head hands on hidden states
            out = CausalLMOutput()
            out.hidden_states = hidden
            return out
        # the head's saved tensors are the first that backward asks for: activation offloading leaves them on the device
        ctx = getattr(self, "head_saved_tensors_ctx", None)
        preshifted = bool(getattr(meta, "labels_preshifted", False))
        if ctx is None:
            return self._head(hidden, labels, return_logits, preshifted)
        with ctx():
            return self._head(hidden, labels, return_logits, preshifted)

    def _head(self, hidden: torch.Tensor, labels: Optional[torch.Tensor], return_logits: Optional[bool],
              preshifted: bool = False) -> CausalLMOutput:
        out = CausalLMOutput()
        if labels is None:
            out.logits = self.lm_head(hidden)
            return out
        # shift: the label of position t is token t+1; the last position of every row has no target
        # (fla/models/transformer/modeling_transformer.py:428).  A context-parallel slice arrives already shifted.
        if preshifted:
            shifted = labels.reshape(-1)
        elif labels.dim() == 2:
            shifted = torch.cat([labels[:, 1:], torch.full_like(labels[:, :1], -100)], 1).reshape(-1)
        else:
            shifted = torch.cat([labels[1:], torch.full_like(labels[:1], -100)], 0)
        tp = getattr(self, "tp", None)
        if tp is not None:
            # sequence-sharded hidden states -> gathered GEMM against the vocabulary shard -> vocabulary-parallel loss
            from ..parallel.tensor_parallel import allgather_linear, vocab_parallel_cross_entropy
            logits = allgather_linear(hidden, (self.lm_head.weight,))
            out.loss = vocab_parallel_cross_entropy(logits, shifted, tp.rank * self.lm_head.weight.shape[0],
                                                    grad_scale=self.loss_grad_scale)
            return out
        fuse = self.config.fuse_linear_cross_entropy or (self.config.fuse_cross_entropy and hidden.is_cuda)
        if fuse and not return_logits:
            out.loss = ce_ops.fused_linear_cross_entropy(hidden, self.lm_head.weight, shifted,
                                                         grad_scale=self.loss_grad_scale)
        else:
            logits = self.lm_head(hidden)
            loss = ce_ops.cross_entropy(logits if not return_logits else logits.clone(), shifted)
            if self.loss_grad_scale != 1.0:  # same value, gradient scaled (gradient accumulation)
                loss = loss.detach() + (loss - loss.detach()) * self.loss_grad_scale
            out.loss = loss
            if return_logits:
                out.logits = logits
        return out

    # -- initialisation ------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: Optional[int] = None) -> None:
        """normal(0, initializer_range) for projections / convolutions / embeddings, zeros for biases, ones for
        norm weights, family-specific values for A_log / dt_bias / D / dt_proj, and the
        ``rescale_prenorm_residual`` scaling of output projections (fla/models/*/modeling_*.py ``_init_weights``).
        Every parameter is drawn on the CPU from one generator so all ranks and world sizes see the same model."""
        base = 0x5EED if seed is None else int(seed)

        def gen_for(name: str) -> torch.Generator:
            # one generator per parameter, keyed by its name: the values do not depend on which other modules exist
            # (pipeline stages) or on the order they are visited in
            import zlib
            g = torch.Generator(device="cpu")
            g.manual_seed((base * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
            return g

        std = self.config.initializer_range
        for name, mod in self.named_modules():
            if isinstance(mod, (Linear, Embedding, ShortConvolution)):
                _normal_(mod.weight, std, gen_for(name + ".weight"))
                if getattr(mod, "bias", None) is not None:
                    mod.bias.zero_()
            elif isinstance(mod, (RMSNorm, L.RMSNormGated)):
                if mod.weight is not None:
                    mod.weight.fill_(1.0)
        for name, mod in self.named_modules():
            if isinstance(mod, L.GatedDeltaNet) or isinstance(mod, L.Mamba2):
                mod.reset_special_parameters(gen_for(name))
            elif isinstance(mod, L.Mamba):
                mod.reset_special_parameters(self.config, gen_for(name))
        dec = self.decoder
        if hasattr(dec, "lower_bounds"):
            dec.lower_bounds.zero_()
        if self.config.get("rescale_prenorm_residual", False):
            n = self.config.num_hidden_layers
            for name, p in self.named_parameters():
                if name.endswith("out_proj.weight") or name.endswith("o_proj.weight") or name.endswith("down_proj.weight"):
                    p.div_(math.sqrt(2 * n) if self.config.model_type != "mamba2" else math.sqrt(n))

    # -- HF-layout persistence -------------------------------------------------------------------------
    def save_pretrained(self, path: str, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                        dtype: Optional[torch.dtype] = None) -> None:
        """Writes ``config.json`` + ``model.safetensors`` (what ``PreTrainedModel.save_pretrained`` produces)."""
        from safetensors.torch import save_file
        os.makedirs(path, exist_ok=True)
        cfg = self.config.to_dict()
        cfg["architectures"] = [ARCHITECTURES.get(self.config.model_type, "CausalLM")]
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2, sort_keys=True)
        sd = state_dict if state_dict is not None else self.state_dict()
        out = {}
        for k, v in sd.items():
            t = v.detach().to("cpu")
            if dtype is not None and t.is_floating_point():
                t = t.to(dtype)
            out[k] = t.contiguous()
        save_file(out, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})

    @classmethod
    def from_pretrained(cls, path: str, device: str = "cpu", dtype: Optional[torch.dtype] = None) -> "CausalLM":
        from safetensors.torch import load_file
        cfg = ModelConfig.from_pretrained(path)
        model = cls(cfg)
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        sd: Dict[str, torch.Tensor] = {}
        if files:
            for f in files:
                sd.update(load_file(os.path.join(path, f)))
        elif os.path.exists(os.path.join(path, "pytorch_model.bin")):
            sd = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True)
        else:
            raise FileNotFoundError(f"no weights under {path}")
        missing, unexpected = model.load_state_dict(sd, strict=False)
        if missing or unexpected:
            raise RuntimeError(f"state dict mismatch: missing={missing[:5]} unexpected={unexpected[:5]}")
        if dtype is not None:
            model = model.to(dtype)
        return model.to(device)

    def num_parameters(self, exclude_embeddings: bool = False) -> int:
        n = sum(p.numel() for p in self.parameters())
        if exclude_embeddings:
            n -= self.decoder.embeddings.weight.numel()
        return n


ARCHITECTURES = {
    "transformer": "TransformerForCausalLM", "sba": "SBAForCausalLM", "gla": "GLAForCausalLM",
    "delta_net": "DeltaNetForCausalLM", "gated_deltanet": "GatedDeltaNetForCausalLM", "gsa": "GSAForCausalLM",
    "hgrn2": "HGRN2ForCausalLM", "mamba": "MambaForCausalLM", "mamba2": "Mamba2ForCausalLM",
    "samba": "SambaForCausalLM",
}


def _normal_(p: torch.Tensor, std: float, gen: torch.Generator) -> None:
    if p.device.type == "meta":
        return
    tp = getattr(p, "_tp", None)
    if tp is not None:
        # tensor-parallel shard: draw the FULL tensor (so every tp degree sees the same model) and keep this rank's slice
        dim, rank, world = tp
        full = list(p.shape)
        full[dim] *= world
        rows = full[0]
        per = max(1, (1 << 24) // max(1, int(torch.tensor(full[1:]).prod()) if len(full) > 1 else 1))
        n_local = p.shape[dim]
        for a in range(0, rows, per):
            b = min(rows, a + per)
            blk = torch.empty([b - a] + full[1:], dtype=torch.float32).normal_(0.0, std, generator=gen)
            if dim == 0:
                lo, hi = max(a, rank * n_local), min(b, (rank + 1) * n_local)
                if lo < hi:
                    p[lo - rank * n_local:hi - rank * n_local].copy_(blk[lo - a:hi - a])
            else:
                p[a:b].copy_(blk.narrow(dim, rank * n_local, n_local))
        return
    # drawn in fp32 on the CPU in row blocks so large embeddings never need a second full-size temporary
    flat = p.view(-1)
    n = flat.numel()
    step = 1 << 24
    for a in range(0, n, step):
        b = min(n, a + step)
        flat[a:b].copy_(torch.empty(b - a, dtype=torch.float32).normal_(0.0, std, generator=gen))


def build_model(cfg: ModelConfig, device: str | torch.device = "cpu", dtype: torch.dtype = torch.float32,
                init: bool = True, seed: Optional[int] = None) -> CausalLM:
    with torch.device(device):
        model = CausalLM(cfg)
    model = model.to(dtype)
    if init and str(device) != "meta":
        model.init_weights(seed)
    return model


def get_blocks(model: CausalLM) -> nn.ModuleList:
    return model.decoder.layers
