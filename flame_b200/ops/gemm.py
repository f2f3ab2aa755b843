"""Dense bf16 matmuls on the tcgen05 GEMM kernel (``csrc/gemm.cu``).

Three forms cover a linear layer's forward, data gradient and weight gradient without any transpose
copy, because the kernel reads either operand K-major or MN-major straight from its row-major storage:

* ``gemm_nt(x, w)``  = ``x @ w.T``    forward            (x [M,K], w [N,K])
* ``gemm_nn(dy, w)`` = ``dy @ w``     data gradient      (dy [M,N], w [N,K])
* ``gemm_tn(dy, x)`` = ``dy.T @ x``   weight gradient    (dy [T,N], x [T,K]) -> [N,K]

They stand in for the cuBLAS calls behind every ``nn.Linear`` of the reference
(fla/modules/mlp.py:58-73, fla/layers/attn.py:73-82).  On a machine without CUDA the same functions
compute with ``torch.matmul`` in the tensors' own dtype; that path is the test oracle's subject on CPU
and the execution path of the CPU/gloo plumbing runs.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

_WORKSPACES: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-device split-K scratch, grown on demand and reused (stream-ordered reuse is safe because
    every consumer runs on the launching stream)."""
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _use_kernel(*ts: torch.Tensor) -> bool:
    return _lib.available() and all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    # kernel needs: inner stride 1, leading dimension a multiple of 8 elements, base 16-byte aligned
    if t.stride(-1) != 1 or (t.stride(0) % 8) != 0 or (t.data_ptr() % 16) != 0:
        t = t.contiguous()
        if t.stride(0) % 8 != 0:
            raise ValueError("bf16 GEMM operands need a row length that is a multiple of 8 elements")
    return t


def _launch(a, b, M, N, K, a_mn, b_mn, out, accumulate, alpha, bias, splits):
    L = _lib.lib()
    a = _rows_ok(a)
    b = _rows_ok(b)
    if out.dtype == torch.bfloat16:
        mode = 0
        if accumulate:
            raise ValueError("accumulation needs an fp32 output")
    elif out.dtype == torch.float32:
        mode = 2 if accumulate else 1
    else:
        raise ValueError(f"unsupported output dtype {out.dtype}")
    if out.stride(-1) != 1:
        raise ValueError("output must be row-major")
    if splits is None:
        splits = int(L.fb_gemm_pick_splits(M, N, K)) if out.stride(0) == N and (M * N) % 4 == 0 else 1
    ws = None
    if splits > 1:
        ws = _workspace(out.device, int(L.fb_gemm_workspace_bytes(M, N, splits)))
    rc = L.fb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                        int(a_mn), int(b_mn), mode, float(alpha), _lib.ptr(bias), int(splits), _lib.ptr(ws),
                        _lib.stream_ptr())
    _lib.check(rc, "fb_gemm_bf16")
    _lib.count_launch(2 if splits > 1 else 1)
    return out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *,
            out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
            bias: Optional[torch.Tensor] = None, splits: Optional[int] = None) -> torch.Tensor:
    """``a [M,K] @ b[N,K].T -> [M,N]``."""
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape)
    if _use_kernel(a, b):
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        return _launch(a, b, M, N, K, 0, 0, out, accumulate, alpha, bias, splits)
    r = torch.matmul(a, b.t())
    if alpha != 1.0:
        r = r * alpha
    if bias is not None:
        r = r + bias
    return _finish(r, out, out_dtype, accumulate)


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *,
            out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
            splits: Optional[int] = None) -> torch.Tensor:
    """``a [M,K] @ b[K,N] -> [M,N]`` with ``b`` row-major (its N dimension contiguous)."""
    M, K = a.shape
    Kb, N = b.shape
    assert K == Kb, (a.shape, b.shape)
    if _use_kernel(a, b):
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        return _launch(a, b, M, N, K, 0, 1, out, accumulate, alpha, None, splits)
    r = torch.matmul(a, b)
    if alpha != 1.0:
        r = r * alpha
    return _finish(r, out, out_dtype, accumulate)


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *,
            out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
            splits: Optional[int] = None) -> torch.Tensor:
    """``a[K,M].T @ b[K,N] -> [M,N]``; the reduction runs over the leading (token) dimension of both."""
    K, M = a.shape
    Kb, N = b.shape
    assert K == Kb, (a.shape, b.shape)
    if _use_kernel(a, b):
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        return _launch(a, b, M, N, K, 1, 1, out, accumulate, alpha, None, splits)
    r = torch.matmul(a.t(), b)
    if alpha != 1.0:
        r = r * alpha
    return _finish(r, out, out_dtype, accumulate)


def _finish(r, out, out_dtype, accumulate):
    if out is None:
        return r.to(out_dtype) if out_dtype is not None else r
    if accumulate:
        out.add_(r.to(out.dtype))
    else:
        out.copy_(r)
    return out
