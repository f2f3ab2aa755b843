"""ctypes binding to the ahead-of-time built sm_100a kernel library.

``lib()`` returns the loaded ``libflame_b200.so``.  On a machine with a CUDA device the library is
mandatory: if it is missing it is built, and if that fails an exception is raised, so a GPU run can never
fall back silently to framework kernels.  On a CPU-only machine ``available()`` is False and the ops in
this package run their PyTorch reference implementations.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _build

_LIB: Optional[ctypes.CDLL] = None
_LAUNCHES = 0
_PEER_WAIT_SECONDS = 2.0


class KernelError(RuntimeError):
    pass


def cuda_present() -> bool:
    return torch.cuda.is_available()


def available() -> bool:
    """True when kernels of this library should be used (a CUDA device is present)."""
    return cuda_present() and os.environ.get("FLAME_B200_FORCE_REFERENCE", "0") != "1"


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not _build.LIB_PATH.exists():
            _build.build_library()
        _LIB = ctypes.CDLL(str(_build.LIB_PATH))
        _declare(_LIB)
    return _LIB


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launches() -> int:
    """Number of kernels of this library launched by this process so far."""
    return _LAUNCHES


def reset_launches() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def status() -> int:
    """Library status word: 0 = ok, otherwise ``code << 16 | block``; see ``csrc/tc05.cuh``."""
    return int(lib().fb_status_read())


def status_clear() -> None:
    lib().fb_status_clear()


_STATUS_CODES = {1: "a TMA stage never landed", 2: "a pipeline stage was never released",
                 3: "an accumulator never completed", 4: "an accumulator was never drained",
                 5: "a flag that another GPU (or CTA) raises never came", 6: "an in-kernel barrier never completed",
                 7: "a kernel rejected an argument"}


def describe_status(s: int) -> str:
    code, detail = s >> 16, s & 0xffff
    what = _STATUS_CODES.get(code, "unknown code")
    who = f"peer rank / flag index {detail}" if code == 5 else f"block {detail}"
    return f"kernel status word is {s:#x} (code {code}: {what}; {who}): a bounded wait ran out"


def assert_status_ok(sync: bool = True) -> None:
    """Raises ``KernelError`` when a kernel recorded a failed wait.  ``sync=False`` only reads the pinned word (no stream
    synchronisation): errors of kernels that are still running are then seen by a later call."""
    if sync:
        torch.cuda.synchronize()
    s = status()
    if s != 0:
        raise KernelError(describe_status(s))


def set_peer_wait_seconds(seconds: float) -> None:
    """Limit of every later device-side wait on a flag that another GPU raises (peer collectives, fused gathers)."""
    global _PEER_WAIT_SECONDS
    _PEER_WAIT_SECONDS = max(1e-3, float(seconds))
    if cuda_present():
        lib().fb_set_peer_wait_seconds(c_double(_PEER_WAIT_SECONDS))


def peer_wait_seconds() -> float:
    return _PEER_WAIT_SECONDS


def _declare(L: ctypes.CDLL) -> None:
    vp, i, ll, f = c_void_p, c_int, c_longlong, c_float
    L.fb_status_read.restype = c_int
    L.fb_status_clear.restype = None
    L.fb_set_peer_wait_seconds.argtypes = [c_double]
    L.fb_set_peer_wait_seconds.restype = None
    sigs = {
        "fb_gemm_bf16": [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, f, vp, i, vp, vp],
        "fb_gemm_pick_splits": [i, i, i],
        "fb_gemm_set_variant": [i],
    }
    for name, args in sigs.items():
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int
    L.fb_gemm_workspace_bytes.argtypes = [i, i, i]
    L.fb_gemm_workspace_bytes.restype = c_longlong
    for name, args, res in _EXTRA_SIGS:
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = res


# (name, argtypes, restype) registered by the op modules before first use of lib()
_EXTRA_SIGS: list = []


def register(name: str, argtypes: list, restype=c_int) -> None:
    _EXTRA_SIGS.append((name, argtypes, restype))
    if _LIB is not None:
        fn = getattr(_LIB, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = restype
