"""Packed-sequence (varlen) metadata shared by every kernel of one batch.

The trainer builds one ``VarlenMeta`` per micro-batch from ``cu_seqlens``; all layers, forward and backward,
reuse it.  On CUDA the derived index arrays are produced by small device kernels (no ``tolist()`` round trip,
unlike fla/ops/utils/index.py:114-156, which builds them on the host and caches them).
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib

_lib.register("fb_position_ids", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p])
_lib.register("fb_attn_tile_offsets", [c_void_p, c_int, c_void_p, c_void_p])


@dataclass
class VarlenMeta:
    cu_seqlens: torch.Tensor  # int32 [nseq + 1] on the compute device
    total_tokens: int
    nseq: int
    max_tiles128: int  # upper bound on the number of 128-token tiles over all documents
    _pos: Optional[torch.Tensor] = None
    _seq_id: Optional[torch.Tensor] = None
    _tile_offsets: Optional[torch.Tensor] = None
    _cu_cpu: Optional[torch.Tensor] = None
    cache: dict = field(default_factory=dict)

    @staticmethod
    def from_cu_seqlens(cu_seqlens: torch.Tensor, total_tokens: Optional[int] = None,
                        device: Optional[torch.device] = None) -> "VarlenMeta":
        cu_cpu = cu_seqlens if cu_seqlens.device.type == "cpu" else None
        device = device or cu_seqlens.device
        cu = cu_seqlens.to(device=device, dtype=torch.int32, non_blocking=True)
        nseq = cu.numel() - 1
        if total_tokens is None:
            total_tokens = int(cu_seqlens[-1])
        return VarlenMeta(cu_seqlens=cu, total_tokens=total_tokens, nseq=nseq,
                          max_tiles128=total_tokens // 128 + nseq, _cu_cpu=cu_cpu)

    @staticmethod
    def dense(batch: int, seq_len: int, device: torch.device) -> "VarlenMeta":
        """Metadata for ``batch`` equal-length rows packed back to back (non-varlen training)."""
        cu = torch.arange(0, (batch + 1) * seq_len, seq_len, dtype=torch.int32)
        return VarlenMeta.from_cu_seqlens(cu, batch * seq_len, device)

    @property
    def device(self) -> torch.device:
        return self.cu_seqlens.device

    def cu_cpu(self) -> torch.Tensor:
        if self._cu_cpu is None:
            self._cu_cpu = self.cu_seqlens.cpu()
        return self._cu_cpu

    def _build_pos(self) -> None:
        T = self.total_tokens
        if self.device.type == "cuda" and _lib.available():
            pos = torch.empty(T, dtype=torch.int32, device=self.device)
            sid = torch.empty(T, dtype=torch.int32, device=self.device)
            rc = _lib.lib().fb_position_ids(self.cu_seqlens.data_ptr(), self.nseq + 1, pos.data_ptr(), sid.data_ptr(), T,
                                            _lib.stream_ptr())
            _lib.check(rc, "fb_position_ids")
            _lib.count_launch()
        else:
            cu = self.cu_seqlens.long()
            lens = cu[1:] - cu[:-1]
            sid = torch.repeat_interleave(torch.arange(self.nseq, device=self.device), lens)
            pos = (torch.arange(T, device=self.device) - cu[:-1][sid]).to(torch.int32)
            sid = sid.to(torch.int32)
        self._pos, self._seq_id = pos, sid

    @property
    def position_ids(self) -> torch.Tensor:
        """int32 [T]: offset of every token inside its document."""
        if self._pos is None:
            self._build_pos()
        return self._pos

    @property
    def seq_ids(self) -> torch.Tensor:
        if self._seq_id is None:
            self._build_pos()
        return self._seq_id

    @property
    def tile_offsets(self) -> torch.Tensor:
        """int32 [nseq + 1]: prefix sum of ``ceil(len / 128)`` (attention work list)."""
        if self._tile_offsets is None:
            if self.device.type == "cuda" and _lib.available():
                t = torch.empty(self.nseq + 1, dtype=torch.int32, device=self.device)
                rc = _lib.lib().fb_attn_tile_offsets(self.cu_seqlens.data_ptr(), self.nseq, t.data_ptr(),
                                                     _lib.stream_ptr())
                _lib.check(rc, "fb_attn_tile_offsets")
                _lib.count_launch()
            else:
                cu = self.cu_seqlens.long()
                n = (cu[1:] - cu[:-1] + 127) // 128
                t = torch.cat([torch.zeros(1, dtype=torch.long, device=self.device), n.cumsum(0)]).to(torch.int32)
            self._tile_offsets = t
        return self._tile_offsets

    def lengths_list(self) -> list[int]:
        cu = self.cu_cpu().tolist()
        return [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
