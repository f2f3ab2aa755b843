"""Operator-level selective activation checkpointing: which op outputs a checkpointed block keeps.

The reference's ``selective`` mode with option ``op`` (flame/models/parallelize_fla.py:284-331) recomputes a block in
backward but keeps the outputs of its expensive operators - every matrix product except each second one, and the
attention - so that the recomputation only re-runs the cheap element-wise and normalisation work around them.  It
gets there through a dispatcher-level policy of the tracing machinery; the kernels here are opaque to the dispatcher,
so the same policy is kept by the operators themselves:

* a checkpointed block runs under a ``Tape``.  The first run (forward) is the *record* pass: an operator asks
  ``decide(kind)`` whether its output is to be kept and, if so, ``store``s it;
* the second run (the recomputation inside backward) is the *replay* pass: the operator ``fetch``es the kept output
  and hands it to its autograd function as the already-known result, so no kernel runs but the node still enters the
  new graph with its inputs saved for backward.

Kinds: ``"mm"`` (``ops.linear``: the 1st, 3rd, ... products of the block are kept, the 2nd, 4th, ... recomputed) and
``"attn"`` (``ops.attention``: output and log-sum-exp, always kept).
"""
from __future__ import annotations

import threading
from typing import Any, List, Optional

_tls = threading.local()


class Tape:
    def __init__(self) -> None:
        self.values: List[Any] = []   # one entry per operator call of the block, None when recomputed
        self.mode: Optional[str] = None
        self.pos = 0
        self.mm_count = 0
        self.runs = 0

    def begin_run(self) -> None:
        """First run records, every later run (the recomputation) replays."""
        self.runs += 1
        self.mode = "record" if self.runs == 1 else "replay"
        self.pos = 0
        self.mm_count = 0

    # -- record pass ---------------------------------------------------------------------------------
    def decide(self, kind: str) -> bool:
        keep = True
        if kind == "mm":
            self.mm_count += 1
            keep = self.mm_count % 2 == 1
        self.values.append(None)
        self._keep = keep
        return keep

    def store(self, value: Any) -> None:
        if self._keep:
            self.values[-1] = value

    # -- replay pass ---------------------------------------------------------------------------------
    def fetch(self) -> Any:
        if self.pos >= len(self.values):
            return None  # the recomputation took another path than the forward: recompute from here on
        v, self.values[self.pos] = self.values[self.pos], None  # release the reference: autograd owns it from now on
        self.pos += 1
        return v

    def kept_bytes(self) -> int:
        n = 0
        for v in self.values:
            for t in (v if isinstance(v, (tuple, list)) else (v,)):
                if hasattr(t, "numel"):
                    n += t.numel() * t.element_size()
        return n


class use:
    """``with use(tape):`` makes ``tape`` the current one on this thread (the recomputation runs on autograd's thread)."""

    def __init__(self, tape: Optional[Tape]) -> None:
        self.tape = tape

    def __enter__(self):
        self.prev = getattr(_tls, "tape", None)
        _tls.tape = self.tape
        return self.tape

    def __exit__(self, *exc):
        _tls.tape = self.prev
        return False


def current() -> Optional[Tape]:
    return getattr(_tls, "tape", None)
