"""Building blocks shared by all model families.  Everything works on packed ``[T, D]`` activations plus the
batch's ``VarlenMeta``; parameter names and shapes are those of the reference's state dict
(``q_proj.weight [out, in]``, ``conv1d.weight [D, 1, W]``, ...), so checkpoints interchange."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from ..ops import activations, linear as linear_ops, norm as norm_ops
from ..ops.embedding import embedding
from ..ops.conv import short_conv
from ..ops.varlen import VarlenMeta


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_ops.linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


def fused_projection(x: torch.Tensor, layers: Sequence[Linear]) -> torch.Tensor:
    """One GEMM for several bias-free projections of the same input; returns their outputs side by side."""
    return linear_ops.linear_fused(x, [l.weight for l in layers])


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        tp = getattr(self, "tp", None)
        if tp is None:
            return embedding(ids, self.weight)
        # vocabulary-parallel: look up the local slice (zeros elsewhere), then reduce-scatter over the token rows
        from ..parallel.tensor_parallel import _ScatterRowsSum
        n = self.weight.shape[0]
        local = ids - tp.rank * n
        from ..ops import _lib
        if _lib.available() and self.weight.is_cuda and self.weight.dtype == torch.bfloat16 and self.weight.shape[1] % 8 == 0:
            # the gather kernel returns zero rows for ids outside [0, n) and its backward skips them, so tokens of other
            # ranks' vocabulary slices neither read nor pile up on one row of the gradient
            out = embedding(local, self.weight)
        else:
            mine = (local >= 0) & (local < n)
            out = embedding(local.clamp(0, n - 1), self.weight) * mine[..., None].to(self.weight.dtype)
        return _ScatterRowsSum.apply(out)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-6) -> None:
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps
        self.weight = nn.Parameter(torch.ones(hidden_size)) if elementwise_affine else None

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, prenorm: bool = False):
        return norm_ops.rms_norm(x, self.weight, self.eps, residual, prenorm)


class RMSNormGated(nn.Module):
    """``norm(x) * weight * act(gate)`` over the last dimension (per-head output norm of the linear-attention layers)."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-6,
                 activation: str = "swish") -> None:
        super().__init__()
        self.hidden_size, self.eps, self.activation = hidden_size, eps, activation
        self.weight = nn.Parameter(torch.ones(hidden_size)) if elementwise_affine else None

    def forward(self, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        return norm_ops.rms_norm_gated(x, gate, self.weight, self.eps, self.activation)


class GatedMLP(nn.Module):
    """SwiGLU MLP: ``down(silu(gate(x)) * up(x))`` with gate and up evaluated by one GEMM."""

    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_proj = Linear(hidden_size, intermediate_size)
        self.up_proj = Linear(hidden_size, intermediate_size)
        self.down_proj = Linear(intermediate_size, hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if getattr(self, "tp", None) is not None:
            from ..parallel.tensor_parallel import allgather_linear, linear_reduce_scatter
            gu = allgather_linear(x, (self.gate_proj.weight, self.up_proj.weight))
            return linear_reduce_scatter(activations.swiglu(gu), self.down_proj.weight)
        from ..ops.linear import gate_up_swiglu
        z = gate_up_swiglu(x, self.gate_proj.weight, self.up_proj.weight)   # activation in the GEMM epilogue (opt-in)
        if z is None:
            z = activations.swiglu(fused_projection(x, (self.gate_proj, self.up_proj)))
        return self.down_proj(z)


class ShortConvolution(nn.Module):
    """Depthwise causal conv over time; parameters laid out like ``nn.Conv1d(D, D, W, groups=D)``."""

    def __init__(self, hidden_size: int, kernel_size: int = 4, bias: bool = False,
                 activation: Optional[str] = "silu") -> None:
        super().__init__()
        self.hidden_size, self.kernel_size, self.activation = hidden_size, kernel_size, activation
        self.weight = nn.Parameter(torch.empty(hidden_size, 1, kernel_size))
        self.bias = nn.Parameter(torch.empty(hidden_size)) if bias else None

    def forward(self, x: torch.Tensor, meta: VarlenMeta) -> torch.Tensor:
        return short_conv(x, self.weight, self.bias, meta, self.activation)
