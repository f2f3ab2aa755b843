"""Token-mixing layers of every supported family, on packed ``[T, D]`` activations.

Each class keeps the parameter names and shapes of its reference counterpart (cited per class) so state dicts
interchange; the computation goes through ``flame_b200.ops``.  ``forward(x, meta)`` returns ``[T, D]``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import linear_attn as la
from ..ops.attn_block import qkv_attention
from ..ops.rope import rope_tables
from ..ops.varlen import VarlenMeta
from .config import ModelConfig, mamba_dt_rank
from .modules import Linear, RMSNorm, RMSNormGated, ShortConvolution, fused_projection


class Attention(nn.Module):
    """Causal softmax attention with RoPE, GQA and optional sliding window (fla/layers/attn.py:34-181)."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: Optional[int] = None, qkv_bias: bool = False,
                 qk_norm: bool = False, window_size: Optional[int] = None, rope_theta: Optional[float] = 10000.0,
                 max_position_embeddings: Optional[int] = None, norm_eps: float = 1e-5) -> None:
        super().__init__()
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = hidden_size // num_heads
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.window_size, self.rope_theta = window_size, rope_theta
        self.max_position_embeddings = max_position_embeddings
        self.q_proj = Linear(hidden_size, hidden_size, bias=qkv_bias)
        self.k_proj = Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.v_proj = Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.o_proj = Linear(hidden_size, hidden_size)
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = RMSNorm(self.head_dim, eps=norm_eps)
            self.k_norm = RMSNorm(self.head_dim, eps=norm_eps)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        tp = getattr(self, "tp", None)
        if tp is not None:
            from ..parallel.tensor_parallel import allgather_linear
            qkv = allgather_linear(x, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
        elif self.q_proj.bias is None:
            qkv = fused_projection(x, (self.q_proj, self.k_proj, self.v_proj))
        else:
            qkv = torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x)], -1)
        T = qkv.shape[0]
        if self.qk_norm:
            q = self.q_norm(qkv[:, : H * Dh].reshape(T, H, Dh)).reshape(T, H * Dh)
            k = self.k_norm(qkv[:, H * Dh: (H + Hkv) * Dh].reshape(T, Hkv, Dh)).reshape(T, Hkv * Dh)
            qkv = torch.cat([q, k, qkv[:, (H + Hkv) * Dh:]], -1)
        rope = None
        if self.rope_theta is not None:
            max_pos = max(int(self.max_position_embeddings or 0), _max_doc_len(meta))
            rope = rope_tables(Dh, max_pos, float(self.rope_theta), x.device)
        o = qkv_attention(qkv, meta, H, Hkv, Dh, rope=rope, window=self.window_size or 0)
        if tp is not None:
            from ..parallel.tensor_parallel import linear_reduce_scatter
            return linear_reduce_scatter(o, self.o_proj.weight)
        return self.o_proj(o)


def _max_doc_len(meta: VarlenMeta) -> int:
    m = meta.cache.get("max_len")
    if m is None:
        m = max(meta.lengths_list()) if meta.nseq > 0 else 1
        meta.cache["max_len"] = m
    return m


class StickBreakingAttention(nn.Module):
    """Stick-breaking attention layer (custom_models/sba/sba_layer.py:35-128): q/k/v/o projections, no RoPE.
    Unlike the reference layer, packed documents (``cu_seqlens``) are supported."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: Optional[int] = None, qkv_bias: bool = False) -> None:
        super().__init__()
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = hidden_size // num_heads
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.q_proj = Linear(hidden_size, hidden_size, bias=qkv_bias)
        self.k_proj = Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.v_proj = Linear(hidden_size, self.kv_dim, bias=qkv_bias)
        self.o_proj = Linear(hidden_size, hidden_size)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.stickbreaking import sb_attention
        T = x.shape[0]
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        if self.q_proj.bias is None:
            qkv = fused_projection(x, (self.q_proj, self.k_proj, self.v_proj))
        else:
            qkv = torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x)], -1)
        q = qkv[:, : H * Dh].view(T, H, Dh)  # strided views of the fused projection output
        k = qkv[:, H * Dh: (H + Hkv) * Dh].view(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        if Hkv != H:
            k = k.repeat_interleave(H // Hkv, 1)
            v = v.repeat_interleave(H // Hkv, 1)
        o, _ = sb_attention(q, k, v, meta)
        return self.o_proj(o.reshape(T, H * Dh))


class GatedLinearAttention(nn.Module):
    """GLA (fla/layers/gla.py:27-302): per-channel forget gate from a low-rank projection, swish output gate."""

    def __init__(self, hidden_size: int, expand_k: float = 0.5, expand_v: float = 1.0, num_heads: int = 4,
                 num_kv_heads: Optional[int] = None, feature_map: Optional[str] = None, use_short_conv: bool = False,
                 conv_size: int = 4, use_output_gate: bool = True, elementwise_affine: bool = True,
                 norm_eps: float = 1e-5, gate_logit_normalizer: int = 16, gate_low_rank_dim: int = 16,
                 clamp_min: Optional[float] = None, fuse_norm: bool = True) -> None:
        super().__init__()
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.num_kv_groups = num_heads // self.num_kv_heads
        self.key_dim, self.value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        self.key_dim_per_group = self.key_dim // self.num_kv_groups
        self.value_dim_per_group = self.value_dim // self.num_kv_groups
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.use_short_conv, self.use_output_gate = use_short_conv, use_output_gate
        self.clamp_min, self.gate_logit_normalizer = clamp_min, gate_logit_normalizer
        self.feature_map = feature_map
        self.q_proj = Linear(hidden_size, self.key_dim)
        self.k_proj = Linear(hidden_size, self.key_dim_per_group)
        self.v_proj = Linear(hidden_size, self.value_dim_per_group)
        if use_output_gate:
            self.g_proj = Linear(hidden_size, self.value_dim)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, activation="silu")
            self.k_conv1d = ShortConvolution(self.key_dim_per_group, conv_size, activation="silu")
            self.v_conv1d = ShortConvolution(self.value_dim_per_group, conv_size, activation="silu")
        self.gk_proj = nn.Sequential(Linear(hidden_size, gate_low_rank_dim), Linear(gate_low_rank_dim, self.key_dim_per_group, bias=True))
        self.o_proj = Linear(self.value_dim, hidden_size)
        self.fuse_norm_and_gate = fuse_norm and use_output_gate
        if self.fuse_norm_and_gate:
            self.g_norm_swish_gate = RMSNormGated(self.head_v_dim, elementwise_affine, norm_eps, "swish")
        else:
            self.g_norm = RMSNorm(self.head_v_dim, elementwise_affine, norm_eps)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.gla import gla
        H, G = self.num_heads, self.num_kv_groups
        tp = getattr(self, "tp", None)
        g_out = None
        if tp is not None:
            # one gathered GEMM for q, k, v, the output gate and the (replicated) low-rank gate projection
            from ..parallel.tensor_parallel import allgather_linear
            ws = [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]
            if self.use_output_gate:
                ws.append(self.g_proj.weight)
            ws.append(self.gk_proj[0].weight)
            fused = allgather_linear(x, ws)
            sizes = [w.shape[0] for w in ws]
            parts = torch.split(fused, sizes, dim=-1)
            q, k, v = parts[0], parts[1], parts[2]
            if self.use_output_gate:
                g_out = parts[3]
            gk = self.gk_proj[1](parts[-1].contiguous())
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
            gk = self.gk_proj(x)
        T = q.shape[0]
        if self.use_short_conv:
            q, k, v = self.q_conv1d(q, meta), self.k_conv1d(k, meta), self.v_conv1d(v, meta)
        q = q.reshape(T, H, self.head_k_dim)
        k = k.reshape(T, self.num_kv_heads, self.head_k_dim)
        gk = gk.reshape(T, self.num_kv_heads, self.head_k_dim)
        v = v.reshape(T, self.num_kv_heads, self.head_v_dim)
        if G > 1:
            k, gk, v = (t.repeat_interleave(G, 1) for t in (k, gk, v))
        gk = F.logsigmoid(gk.float()) / self.gate_logit_normalizer
        if self.clamp_min is not None:
            gk = gk.clamp_min(self.clamp_min)
        if self.feature_map is not None:
            q, k = _feature_map(self.feature_map, q), _feature_map(self.feature_map, k)
        o = gla(q, k, v, gk, meta)
        if self.use_output_gate:
            g = g_out if g_out is not None else self.g_proj(x)
            if self.fuse_norm_and_gate:
                o = self.g_norm_swish_gate(o.contiguous(), g.reshape(T, H, self.head_v_dim).contiguous()).reshape(T, self.value_dim)
            else:
                o = self.g_norm(o).reshape(T, self.value_dim) * F.silu(g)
        else:
            o = self.g_norm(o).reshape(T, self.value_dim)
        if tp is not None:
            from ..parallel.tensor_parallel import linear_reduce_scatter
            return linear_reduce_scatter(o, self.o_proj.weight)
        return self.o_proj(o)


def _feature_map(name: str, x: torch.Tensor) -> torch.Tensor:
    if name in ("swish", "silu"):
        return F.silu(x)
    if name == "relu":
        return F.relu(x)
    raise NotImplementedError(f"feature map {name!r}")


class DeltaNet(nn.Module):
    """DeltaNet (fla/layers/delta_net.py:36-292): short conv + SiLU on q/k/v, L2-normalised q/k, beta = sigmoid."""

    def __init__(self, hidden_size: int, expand_k: float = 1.0, expand_v: float = 1.0, num_heads: int = 16,
                 use_beta: bool = True, use_gate: bool = False, use_short_conv: bool = True, conv_size: int = 4,
                 qk_activation: str = "silu", qk_norm: str = "l2", allow_neg_eigval: bool = False,
                 norm_eps: float = 1e-5) -> None:
        super().__init__()
        self.num_heads = num_heads
        self.key_dim, self.value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.use_beta, self.use_gate, self.use_short_conv = use_beta, use_gate, use_short_conv
        self.qk_activation, self.qk_norm, self.allow_neg_eigval = qk_activation, qk_norm, allow_neg_eigval
        self.q_proj = Linear(hidden_size, self.key_dim)
        self.k_proj = Linear(hidden_size, self.key_dim)
        self.v_proj = Linear(hidden_size, self.value_dim)
        if use_beta:
            self.b_proj = Linear(hidden_size, num_heads)
        if use_short_conv:
            act = "silu" if qk_activation == "silu" else None
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, activation=act)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, activation=act)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, activation="silu")
        if use_gate:
            self.g_proj = Linear(hidden_size, self.value_dim)
            self.o_norm = RMSNormGated(self.head_v_dim, eps=norm_eps)
        else:
            self.o_norm = RMSNorm(self.head_v_dim, eps=norm_eps)
        self.o_proj = Linear(self.value_dim, hidden_size)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.delta_rule import gated_delta_rule
        T, H = x.shape[0], self.num_heads
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.use_short_conv:
            q, k, v = self.q_conv1d(q, meta), self.k_conv1d(k, meta), self.v_conv1d(v, meta)
        else:
            if self.qk_activation == "silu":
                q, k = F.silu(q), F.silu(k)
            v = F.silu(v)
        q, k = q.reshape(T, H, self.head_k_dim), k.reshape(T, H, self.head_k_dim)
        v = v.reshape(T, H, self.head_v_dim)
        if self.qk_activation == "relu":
            q, k = q.relu(), k.relu()
        elif self.qk_activation == "elu":
            q, k = F.elu(q) + 1, F.elu(k) + 1
        if self.qk_norm == "sum":
            q, k = q / q.sum(-1, keepdim=True), k / k.sum(-1, keepdim=True)
        beta = self.b_proj(x).float().sigmoid() if self.use_beta else torch.ones(T, H, device=x.device)
        if self.allow_neg_eigval:
            beta = beta * 2.0
        o = gated_delta_rule(q, k, v, beta, None, meta, l2norm_qk=(self.qk_norm == "l2"))
        if self.use_gate:
            o = self.o_norm(o, self.g_proj(x).reshape(T, H, self.head_v_dim))
        else:
            o = self.o_norm(o)
        return self.o_proj(o.reshape(T, self.value_dim))


class GatedDeltaNet(nn.Module):
    """Gated DeltaNet (fla/layers/gated_deltanet.py:42-316): decay g = -exp(A_log) softplus(a + dt_bias)."""

    def __init__(self, hidden_size: int, expand_v: float = 2.0, head_dim: int = 256, num_heads: int = 6,
                 num_v_heads: Optional[int] = None, use_gate: bool = True, use_short_conv: bool = True,
                 conv_size: int = 4, allow_neg_eigval: bool = False, norm_eps: float = 1e-5) -> None:
        super().__init__()
        self.num_heads = num_heads
        self.num_v_heads = num_v_heads or num_heads
        self.head_k_dim = head_dim
        self.head_v_dim = int(head_dim * expand_v)
        self.key_dim = num_heads * head_dim
        self.value_dim = self.num_v_heads * self.head_v_dim
        self.use_gate, self.use_short_conv, self.allow_neg_eigval = use_gate, use_short_conv, allow_neg_eigval
        self.q_proj = Linear(hidden_size, self.key_dim)
        self.k_proj = Linear(hidden_size, self.key_dim)
        self.v_proj = Linear(hidden_size, self.value_dim)
        self.a_proj = Linear(hidden_size, self.num_v_heads)
        self.b_proj = Linear(hidden_size, self.num_v_heads)
        self.A_log = nn.Parameter(torch.empty(self.num_v_heads))
        self.dt_bias = nn.Parameter(torch.empty(self.num_v_heads))
        self.A_log._no_weight_decay = True
        self.dt_bias._no_weight_decay = True
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, activation="silu")
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, activation="silu")
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, activation="silu")
        if use_gate:
            self.g_proj = Linear(hidden_size, self.value_dim)
            self.o_norm = RMSNormGated(self.head_v_dim, eps=norm_eps)
        else:
            self.o_norm = RMSNorm(self.head_v_dim, eps=norm_eps)
        self.o_proj = Linear(self.value_dim, hidden_size)

    def reset_special_parameters(self, generator: Optional[torch.Generator] = None) -> None:
        """A ~ U(0, 16), dt log-uniform in [1e-3, 1e-1] stored through the inverse softplus
        (fla/layers/gated_deltanet.py:148-167)."""
        n = self.num_v_heads
        dev = self.A_log.device
        A = torch.empty(n, dtype=torch.float32).uniform_(0, 16, generator=generator).clamp_min(1e-4)
        dt = torch.exp(torch.rand(n, generator=generator) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        dt = dt.clamp(min=1e-4)
        with torch.no_grad():
            self.A_log.copy_(torch.log(A).to(dev))
            self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(dev))

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.delta_rule import gated_delta_rule
        T = x.shape[0]
        H, HV = self.num_heads, self.num_v_heads
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.use_short_conv:
            q, k, v = self.q_conv1d(q, meta), self.k_conv1d(k, meta), self.v_conv1d(v, meta)
        else:
            q, k, v = F.silu(q), F.silu(k), F.silu(v)
        q, k = q.reshape(T, H, self.head_k_dim), k.reshape(T, H, self.head_k_dim)
        v = v.reshape(T, HV, self.head_v_dim)
        if HV > H:
            q, k = q.repeat_interleave(HV // H, 1), k.repeat_interleave(HV // H, 1)
        beta = self.b_proj(x).float().sigmoid()
        if self.allow_neg_eigval:
            beta = beta * 2.0
        g = la.gdn_gate(self.a_proj(x), self.A_log, self.dt_bias)
        o = gated_delta_rule(q, k, v, beta, g, meta, l2norm_qk=True)
        if self.use_gate:
            o = self.o_norm(o, self.g_proj(x).reshape(T, HV, self.head_v_dim))
        else:
            o = self.o_norm(o)
        return self.o_proj(o.reshape(T, self.value_dim))


class GatedSlotAttention(nn.Module):
    """GSA (fla/layers/gsa.py:31-242): keys write into ``num_slots`` memory slots, softmax over slots reads values."""

    def __init__(self, hidden_size: int, expand_k: float = 1.0, expand_v: float = 1.0, num_heads: int = 4,
                 num_kv_heads: Optional[int] = None, num_slots: Optional[int] = 64, feature_map: str = "swish",
                 use_short_conv: bool = False, conv_size: int = 4, elementwise_affine: bool = True,
                 norm_eps: float = 1e-5, gate_logit_normalizer: int = 8, scale: Optional[float] = 1.0) -> None:
        super().__init__()
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.num_kv_groups = num_heads // self.num_kv_heads
        self.key_dim, self.value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        self.key_dim_per_group = self.key_dim // self.num_kv_groups
        self.value_dim_per_group = self.value_dim // self.num_kv_groups
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.num_slots = num_slots or self.head_k_dim
        self.feature_map, self.use_short_conv = feature_map, use_short_conv
        self.gate_logit_normalizer, self.scale = gate_logit_normalizer, scale
        self.q_proj = Linear(hidden_size, self.key_dim)
        self.k_proj = Linear(hidden_size, self.key_dim_per_group)
        self.v_proj = Linear(hidden_size, self.value_dim_per_group)
        self.f_proj = Linear(hidden_size, self.num_kv_heads * self.num_slots)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, activation="silu")
            self.k_conv1d = ShortConvolution(self.key_dim_per_group, conv_size, activation="silu")
            self.v_conv1d = ShortConvolution(self.value_dim_per_group, conv_size, activation="silu")
        self.g_norm = RMSNorm(hidden_size, elementwise_affine, norm_eps)
        self.o_proj = Linear(self.value_dim, hidden_size)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.gla import gsa
        T, H, G = x.shape[0], self.num_heads, self.num_kv_groups
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.use_short_conv:
            q, k, v = self.q_conv1d(q, meta), self.k_conv1d(k, meta), self.v_conv1d(v, meta)
        f = self.f_proj(x)
        q = q.reshape(T, H, self.head_k_dim)
        k = k.reshape(T, self.num_kv_heads, self.head_k_dim)
        v = v.reshape(T, self.num_kv_heads, self.head_v_dim)
        f = f.reshape(T, self.num_kv_heads, self.num_slots)
        q, k = _feature_map(self.feature_map, q), _feature_map(self.feature_map, k)
        v = F.silu(v)
        f = F.logsigmoid(f.float()) / self.gate_logit_normalizer
        s = 1 - f.exp()
        if G > 1:
            k, v, f, s = (t.repeat_interleave(G, 1) for t in (k, v, f, s))
        o = gsa(q, k, v, s, f, meta, scale=self.scale)
        o = self.g_norm(F.silu(o.reshape(T, self.value_dim)))
        return self.o_proj(o)


class HGRN2Attention(nn.Module):
    """HGRN2 (fla/layers/hgrn2.py:29-215): GLA with k = 1 - forget gate and an optional per-layer lower bound."""

    def __init__(self, hidden_size: int, num_heads: int = 8, expand_ratio: int = 128, use_short_conv: bool = False,
                 conv_size: int = 4, elementwise_affine: bool = True, norm_eps: float = 1e-5, layer_idx: int = 0) -> None:
        super().__init__()
        # the head count follows from the expand ratio when one is given, whatever ``num_heads`` says
        # (fla/layers/hgrn2.py:48-53)
        if expand_ratio is not None:
            num_heads = hidden_size // expand_ratio
        elif num_heads is not None:
            expand_ratio = hidden_size // num_heads
        else:
            raise RuntimeError("One of `expand_ratio` or `num_heads` should be provided.")
        self.num_heads, self.expand_ratio, self.layer_idx = num_heads, expand_ratio, layer_idx
        self.forget_dim = num_heads * expand_ratio
        self.input_dim = hidden_size
        self.head_f_dim, self.head_i_dim = expand_ratio, hidden_size // num_heads
        self.use_short_conv = use_short_conv
        self.q_proj = Linear(hidden_size, self.forget_dim)
        self.f_proj = Linear(hidden_size, self.forget_dim)
        self.i_proj = Linear(hidden_size, self.input_dim)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.forget_dim, conv_size, activation=None)
            self.f_conv1d = ShortConvolution(self.forget_dim, conv_size, activation=None)
            self.i_conv1d = ShortConvolution(self.input_dim, conv_size, activation=None)
        self.g_norm = RMSNorm(hidden_size, elementwise_affine, norm_eps)
        self.o_proj = Linear(self.input_dim, hidden_size)

    def forward(self, x: torch.Tensor, meta: VarlenMeta, lower_bound: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..ops.gla import gla
        T, H = x.shape[0], self.num_heads
        q, f, i = self.q_proj(x), self.f_proj(x), self.i_proj(x)
        if self.use_short_conv:
            q, f, i = self.q_conv1d(q, meta), self.f_conv1d(f, meta), self.i_conv1d(i, meta)
        from ..ops.gates import hgrn2_gates
        q, k, g = hgrn2_gates(q, f, lower_bound if (lower_bound is not None and self.layer_idx > 0) else None)
        q, k, g = (t.reshape(T, H, self.head_f_dim) for t in (q, k, g))
        o = gla(q, k, i.reshape(T, H, self.head_i_dim), g, meta)
        return self.o_proj(self.g_norm(o.reshape(T, self.input_dim)))


class Mamba(nn.Module):
    """Mamba-1 mixer (fla/layers/mamba.py:40-397): in_proj -> conv + SiLU -> x_proj -> dt_proj -> selective scan."""

    def __init__(self, hidden_size: int, state_size: int = 16, conv_kernel: int = 4, intermediate_size: int = 2048,
                 time_step_rank: int = 64, use_bias: bool = False, use_conv_bias: bool = True) -> None:
        super().__init__()
        self.hidden_size, self.ssm_state_size, self.intermediate_size = hidden_size, state_size, intermediate_size
        self.time_step_rank, self.conv_kernel_size = time_step_rank, conv_kernel
        self.conv1d = ShortConvolution(intermediate_size, conv_kernel, bias=use_conv_bias, activation="silu")
        self.in_proj = Linear(hidden_size, intermediate_size * 2, bias=use_bias)
        self.x_proj = Linear(intermediate_size, time_step_rank + state_size * 2)
        self.dt_proj = Linear(time_step_rank, intermediate_size, bias=True)
        self.A_log = nn.Parameter(torch.empty(intermediate_size, state_size))
        self.D = nn.Parameter(torch.empty(intermediate_size))
        self.A_log._no_weight_decay = True
        self.D._no_weight_decay = True
        self.out_proj = Linear(intermediate_size, hidden_size, bias=use_bias)

    def reset_special_parameters(self, cfg: ModelConfig, generator: Optional[torch.Generator] = None) -> None:
        """A = arange(1..N) per channel, D = 1, dt_proj so that softplus(bias) is log-uniform in [dt_min, dt_max]
        (fla/models/mamba/modeling_mamba.py:117-147)."""
        Di, N, R = self.intermediate_size, self.ssm_state_size, self.time_step_rank
        dev = self.A_log.device
        scale = cfg.get("dt_scale", cfg.get("time_step_scale", 1.0))
        dt_min = cfg.get("dt_min", cfg.get("time_step_min", 0.001))
        dt_max = cfg.get("dt_max", cfg.get("time_step_max", 0.1))
        floor = cfg.get("dt_init_floor", cfg.get("time_step_floor", 1e-4))
        std = R ** -0.5 * scale
        with torch.no_grad():
            self.A_log.copy_(torch.log(torch.arange(1, N + 1, dtype=torch.float32))[None, :].expand(Di, N).to(dev))
            self.D.fill_(1.0)
            w = torch.empty(Di, R).uniform_(-std, std, generator=generator)
            self.dt_proj.weight.copy_(w.to(dev))
            dt = torch.exp(torch.rand(Di, generator=generator) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
            dt = dt.clamp(min=floor)
            self.dt_proj.bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(dev))

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.scan import selective_scan
        Di, N, R = self.intermediate_size, self.ssm_state_size, self.time_step_rank
        xz = self.in_proj(x)
        h, z = xz[:, :Di], xz[:, Di:]
        h = self.conv1d(h.contiguous(), meta)
        ssm = self.x_proj(h)
        dt, B, C = ssm[:, :R], ssm[:, R:R + N], ssm[:, R + N:]
        delta = F.softplus(self.dt_proj(dt.contiguous()).float())
        A = -torch.exp(self.A_log.float())
        y = selective_scan(h, delta, A, B, C, self.D, meta)
        y = y * F.silu(z)
        return self.out_proj(y.to(x.dtype))


class Mamba2(nn.Module):
    """Mamba-2 mixer (fla/layers/mamba2.py:92-669): in_proj -> (gate, xBC, dt); conv + SiLU on xBC; SSD; gated RMSNorm."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int = 64, state_size: int = 128, expand: int = 2,
                 n_groups: int = 1, conv_kernel: int = 4, use_conv_bias: bool = True, use_bias: bool = False,
                 rmsnorm: bool = True, norm_before_gate: bool = False, norm_eps: float = 1e-5, chunk_size: int = 256,
                 A_init_range=(1, 16), dt_min: float = 0.001, dt_max: float = 0.1, dt_init_floor: float = 1e-4) -> None:
        super().__init__()
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.ssm_state_size, self.n_groups = state_size, n_groups
        self.intermediate_size = int(expand * hidden_size)
        self.conv_dim = self.intermediate_size + 2 * n_groups * state_size
        self.rmsnorm, self.norm_before_gate, self.norm_eps = rmsnorm, norm_before_gate, norm_eps
        self.A_init_range, self.dt_min, self.dt_max, self.dt_init_floor = A_init_range, dt_min, dt_max, dt_init_floor
        self.conv1d = ShortConvolution(self.conv_dim, conv_kernel, bias=use_conv_bias, activation="silu")
        self.in_proj = Linear(hidden_size, self.intermediate_size + self.conv_dim + num_heads, bias=use_bias)
        self.dt_bias = nn.Parameter(torch.empty(num_heads))
        self.A_log = nn.Parameter(torch.empty(num_heads))
        self.D = nn.Parameter(torch.empty(num_heads))
        for p in (self.dt_bias, self.A_log, self.D):
            p._no_weight_decay = True
        if rmsnorm:
            self.norm = RMSNorm(self.intermediate_size, eps=norm_eps)
        self.out_proj = Linear(self.intermediate_size, hidden_size, bias=use_bias)

    def reset_special_parameters(self, generator: Optional[torch.Generator] = None) -> None:
        n, dev = self.num_heads, self.A_log.device
        dt = torch.exp(torch.rand(n, generator=generator) * (math.log(self.dt_max) - math.log(self.dt_min)) + math.log(self.dt_min))
        dt = dt.clamp(min=self.dt_init_floor)
        A = torch.empty(n, dtype=torch.float32).uniform_(*self.A_init_range, generator=generator)
        with torch.no_grad():
            self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(dev))
            self.A_log.copy_(torch.log(A).to(dev))
            self.D.fill_(1.0)

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        from ..ops.scan import mamba2_ssd
        T = x.shape[0]
        Di, H, P, G, N = self.intermediate_size, self.num_heads, self.head_dim, self.n_groups, self.ssm_state_size
        from ..ops import gates
        zxbcdt = self.in_proj(x)
        # column blocks as views whose gradients are written side by side in one pass
        z, xBC, dt = gates.split_columns(zxbcdt, (Di, self.conv_dim, zxbcdt.shape[1] - Di - self.conv_dim))
        xBC = self.conv1d(xBC.contiguous(), meta)
        xs, B, C = gates.split_columns(xBC, (Di, G * N, G * N))
        if not (self.rmsnorm and self.norm_before_gate):
            # everything elementwise around the SSD core in two kernels: dt = softplus(dt + bias), the log decay and
            # x dt before it; the D skip and the silu(z) gate after it
            from ..ops.gla import scalar_gla
            xv, _, g = gates.mamba2_pre(xs, dt, self.dt_bias, self.A_log, H, P)
            y = scalar_gla(C.reshape(T, G, N), B.reshape(T, G, N), xv, g, meta, scale=1.0)
            y = gates.mamba2_post(y, xs, z, self.D, H, P)
            if self.rmsnorm:
                y = _group_rms(y, self.norm.weight, self.norm_eps, G)
            return self.out_proj(y.to(x.dtype))
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        y = mamba2_ssd(xs.reshape(T, H, P), dt, A, B.reshape(T, G, N), C.reshape(T, G, N), self.D, meta)
        y = _group_rms(y.reshape(T, Di), self.norm.weight, self.norm_eps, G) * F.silu(z)
        return self.out_proj(y.to(x.dtype))


def _group_rms(y: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    if groups == 1:
        from ..ops.norm import rms_norm
        return rms_norm(y.contiguous(), w, eps)
    T, D = y.shape
    yf = y.float().reshape(T, groups, D // groups)
    yf = yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps)
    return (yf.reshape(T, D) * w.float()).to(y.dtype)
