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

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _lib

_WORKSPACES: dict = {}


class PendingGather:
    """A unit of sharded parameters whose bytes ``[lo, hi)`` have not been fetched into the staging buffer yet.  The first
    eligible GEMM whose B operand lies in that range fetches them as part of its own launch (``fb_gemm2_gather_b``: copy
    CTAs pull the peers' shards while the MMA CTAs start on the weight rows that have landed); ``flush`` fetches them
    with the stand-alone kernel instead."""

    def __init__(self, unit, dst_ptr: int, lo: int, hi: int, shard_ptrs, world: int, rank: int, shard_bytes: int,
                 chunk_shift: int, flags: torch.Tensor, epoch: int, flush) -> None:
        self.unit, self.dst_ptr, self.lo, self.hi = unit, dst_ptr, lo, hi
        self.shard_ptrs, self.world, self.rank, self.shard_bytes = shard_ptrs, world, rank, shard_bytes
        self.chunk_shift, self.flags, self.epoch, self.flush = chunk_shift, flags, epoch, flush
        self.done = False
        self.fused_launches = 0

    def covers(self, t: torch.Tensor) -> bool:
        p0 = t.data_ptr()
        p1 = p0 + ((t.shape[0] - 1) * t.stride(0) + t.shape[1]) * t.element_size()
        return self.dst_ptr + self.lo <= p0 and p1 <= self.dst_ptr + self.hi

    def touches(self, t: torch.Tensor) -> bool:
        p0 = t.data_ptr()
        return self.dst_ptr <= p0 < self.dst_ptr + self.hi


_PENDING: Optional[PendingGather] = None
_SM_COUNT: dict = {}
_lib.register("fb_gemm2_gather_b", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                                    c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_longlong, c_longlong, c_int,
                                    c_void_p, c_int, c_int, c_void_p])


def set_pending_gather(p: Optional[PendingGather]) -> None:
    global _PENDING
    _PENDING = p


def pending_gather() -> Optional[PendingGather]:
    return _PENDING


def _sm_count(device: torch.device) -> int:
    n = _SM_COUNT.get(device.index)
    if n is None:
        n = _SM_COUNT[device.index] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


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
    pend = _PENDING
    if pend is not None and not pend.done:
        if (mode == 0 and not a_mn and bias is None and alpha == 1.0 and splits in (None, 1) and pend.covers(b)
                and b.stride(0) % 8 == 0):
            rc = L.fb_gemm2_gather_b(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                     out.stride(0), int(b_mn), pend.shard_ptrs.ctypes.data, pend.world, pend.rank,
                                     pend.shard_bytes, pend.dst_ptr, pend.lo, pend.hi, pend.chunk_shift,
                                     pend.flags.data_ptr(), pend.epoch, _sm_count(out.device), _lib.stream_ptr())
            _lib.check(rc, "fb_gemm2_gather_b")
            _lib.count_launch()
            pend.done = True
            pend.fused_launches += 1
            set_pending_gather(None)
            return out
        if pend.touches(a) or pend.touches(b):
            pend.flush()  # this product reads the unit but cannot carry the gather: fetch with the stand-alone kernel
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
