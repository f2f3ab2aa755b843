"""Activation offloading: tensors saved for backward move to pinned host memory during the forward pass and come back
shortly before backward needs them.

Enabled with ``--activation_offload.mode full``.  The roles are those of the reference's hook manager
(flame/models/activation_offloading.py:139-380, which the reference ships but never wires into its trainer):

* a ``saved_tensors_hooks`` pair; tensors below ``min_offload_size`` bytes, parameters and views of parameters stay put;
* device-to-host copies run on a side stream.  The device copy of an activation has to stay alive until its copy has
  finished: at most ``max_fwd_stash_size`` such tensors are kept (the *forward stash*); when the stash is full the
  compute stream is made to wait for the oldest copy (an event wait on the device, never a host synchronisation) and
  that tensor is released;
* in backward the tensors come back in reverse order of packing, so when tensor ``k`` is asked for, the copies of
  ``k - 1 .. k - prefetch`` are issued as well (the *backward prefetch*); the compute stream waits only for ``k``'s event.
  Returned tensors are tied to the compute stream with ``record_stream`` so the allocator cannot hand their memory out
  while a kernel may still read them;
* ``NoOpManager`` switches the hooks off for a region - the output head, whose saved tensors are consumed first in
  backward, so moving them out and straight back would only cost bandwidth.

Nothing here blocks the host: ordering is by stream and event waits only.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, Optional

import torch


class NoOpManager(torch.autograd.graph.saved_tensors_hooks):
    """Inside this context saved tensors are left alone, whatever hooks are active outside (the innermost pair of
    ``saved_tensors_hooks`` wins)."""

    def __init__(self) -> None:
        super().__init__(lambda t: t, lambda t: t)


class _Record:
    __slots__ = ("host", "d2h", "dev", "h2d", "shape")

    def __init__(self, host, d2h) -> None:
        self.host, self.d2h, self.dev, self.h2d = host, d2h, None, None


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    def __init__(self, device: torch.device, min_offload_size: int = 1024, max_fwd_stash_size: int = 5,
                 prefetch: int = 2, use_pin_memory: bool = True) -> None:
        if max_fwd_stash_size < 1:
            raise ValueError(f"max_fwd_stash_size should be at least 1 but is {max_fwd_stash_size}")
        self.device = device
        self.min_bytes = min_offload_size
        self.max_fwd_stash_size = max_fwd_stash_size
        self.prefetch = max(0, prefetch)
        self.use_pin_memory = use_pin_memory
        self.stream = torch.cuda.Stream(device=device)
        self.fwd_stash: "OrderedDict[int, tuple]" = OrderedDict()  # id -> (event, device tensor kept alive)
        self.records: Dict[int, _Record] = {}
        self.next_id = 0
        # counters (read by tests and the memory log)
        self.offloaded_bytes = 0
        self.offloaded_tensors = 0
        self.prefetched = 0
        self.max_stash_seen = 0
        super().__init__(self._pack, self._unpack)

    # ---- forward --------------------------------------------------------------------------------------------
    def _skip(self, t: torch.Tensor) -> bool:
        if not t.is_cuda or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < self.min_bytes:
            return True
        base = t._base if t._base is not None else t
        if isinstance(base, torch.nn.Parameter) or getattr(base, "main_grad", None) is not None:
            return True
        return t.requires_grad and t.is_leaf

    def _pack(self, t: torch.Tensor) -> Any:
        if self._skip(t):
            return t
        cur = torch.cuda.current_stream(self.device)
        # release what has finished copying; if the stash is still full, order the compute stream behind the oldest copy
        for k in [k for k, (ev, _) in self.fwd_stash.items() if ev.query()]:
            del self.fwd_stash[k]
        while len(self.fwd_stash) >= self.max_fwd_stash_size:
            _, (ev, _) = self.fwd_stash.popitem(last=False)
            cur.wait_event(ev)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.use_pin_memory)
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        tid = self.next_id
        self.next_id += 1
        self.fwd_stash[tid] = (ev, t)
        self.max_stash_seen = max(self.max_stash_seen, len(self.fwd_stash))
        self.records[tid] = _Record(host, ev)
        self.offloaded_bytes += t.numel() * t.element_size()
        self.offloaded_tensors += 1
        return ("offloaded", tid)

    # ---- backward -------------------------------------------------------------------------------------------
    def _bring_back(self, tid: int) -> None:
        rec = self.records.get(tid)
        if rec is None or rec.dev is not None:
            return
        with torch.cuda.stream(self.stream):
            # the side stream is in order: this copy runs after the device-to-host copy of the same tensor
            rec.dev = rec.host.to(self.device, non_blocking=True)
            rec.h2d = torch.cuda.Event()
            rec.h2d.record(self.stream)

    def _unpack(self, obj: Any) -> torch.Tensor:
        if not (isinstance(obj, tuple) and len(obj) == 2 and obj[0] == "offloaded"):
            return obj
        tid = obj[1]
        self.fwd_stash.pop(tid, None)
        if tid not in self.records:
            raise RuntimeError("an offloaded activation was asked for twice; keep the graph (retain_graph) is not supported")
        self._bring_back(tid)
        for k in range(tid - 1, tid - 1 - self.prefetch, -1):  # backward walks the tensors in reverse order of packing
            if k in self.records and self.records[k].dev is None:
                self._bring_back(k)
                self.prefetched += 1
        rec = self.records.pop(tid)
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(rec.h2d)
        rec.dev.record_stream(cur)
        return rec.dev

    def reset(self) -> None:
        """Drops everything that was never asked for (a forward without backward) before the next step."""
        self.fwd_stash.clear()
        self.records.clear()


def enable_activation_offload(runner, max_fwd_stash_size: int = 5, min_offload_size: int = 1024) -> Optional[OffloadActivations]:
    """Wraps ``runner.forward_backward`` so every micro-batch runs under the offloading hooks (CUDA only) and exempts
    the model's output head from them."""
    if runner.device.type != "cuda":
        return None
    ctx = OffloadActivations(runner.device, min_offload_size=min_offload_size, max_fwd_stash_size=max_fwd_stash_size)
    inner = runner.forward_backward
    runner.model.head_saved_tensors_ctx = NoOpManager

    def wrapped(batch, loss_scale=1.0):
        ctx.reset()
        with ctx:
            return inner(batch, loss_scale)

    runner.forward_backward = wrapped
    runner.activation_offload = ctx
    return ctx
