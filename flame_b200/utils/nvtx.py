"""NVTX ranges around the phases of a training step, so that a timeline tool shows data loading, forward+backward
(with the overlapped gradient reduce-scatter) and the optimizer as named spans.  A no-op without CUDA."""
from __future__ import annotations

from contextlib import contextmanager

import torch


@contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
