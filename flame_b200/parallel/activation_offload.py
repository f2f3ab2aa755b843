"""Activation offloading: tensors saved for backward move to pinned host memory during the forward pass and come back
just before they are needed.

Enabled with ``--activation_offload.mode full``.  Same idea as the reference's hook manager
(flame/models/activation_offloading.py:30-447, which the reference never wires into its trainer): a
``saved_tensors_hooks`` pair, copies on a side stream, a small-tensor cut-off (1 KiB), parameters and tensors that
are views of parameters stay on the device.  Device copies are released as soon as their device-to-host copy has
finished; the host-to-device copy in backward is issued on the side stream and the compute stream waits on its event.
"""
from __future__ import annotations

from collections import deque
from typing import Any

import torch

MIN_BYTES = 1024


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    def __init__(self, device: torch.device, min_bytes: int = MIN_BYTES) -> None:
        self.device = device
        self.min_bytes = min_bytes
        self.stream = torch.cuda.Stream(device=device)
        self.inflight: deque = deque()  # (event, device tensor kept alive until the copy is done)
        self.offloaded_bytes = 0

        def pack(t: torch.Tensor) -> Any:
            if (not t.is_cuda) or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < self.min_bytes \
                    or getattr(t._base, "main_grad", None) is not None or t.requires_grad and t.is_leaf:
                return t
            while self.inflight and self.inflight[0][0].query():
                self.inflight.popleft()
            self.stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(self.stream):
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                host.copy_(t, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.inflight.append((ev, t))
            self.offloaded_bytes += t.numel() * t.element_size()
            return ("offloaded", host, ev)

        def unpack(obj: Any) -> torch.Tensor:
            if not (isinstance(obj, tuple) and len(obj) == 3 and obj[0] == "offloaded"):
                return obj
            _, host, ev = obj
            ev.synchronize()
            with torch.cuda.stream(self.stream):
                dev_t = host.to(device, non_blocking=True)
                back = torch.cuda.Event()
                back.record(self.stream)
            torch.cuda.current_stream(device).wait_event(back)
            dev_t.record_stream(torch.cuda.current_stream(device))
            return dev_t

        super().__init__(pack, unpack)


def enable_activation_offload(runner) -> None:
    """Wraps ``runner.forward_backward`` so every micro-batch runs under the offloading hooks (CUDA only)."""
    if runner.device.type != "cuda":
        return
    ctx = OffloadActivations(runner.device)
    inner = runner.forward_backward

    def wrapped(batch, loss_scale=1.0):
        with ctx:
            return inner(batch, loss_scale)

    runner.forward_backward = wrapped
    runner.activation_offload = ctx
