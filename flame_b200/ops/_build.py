"""Ahead-of-time build of the sm_100a kernel library.

All CUDA sources under ``flame_b200/csrc`` are compiled by ``nvcc`` into one shared object,
``flame_b200/_lib/libflame_b200.so``, which exports plain C entry points (raw device pointers plus a
``cudaStream_t``).  There is no JIT and no torch C++ header dependency, so a full rebuild takes seconds
and cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
CSRC = PKG_ROOT / "csrc"
LIB_DIR = PKG_ROOT / "_lib"
LIB_PATH = LIB_DIR / "libflame_b200.so"
STAMP_PATH = LIB_DIR / "libflame_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-O3",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def source_files() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == _digest()


def build_library(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile every ``.cu`` file to an object (in parallel) and link the shared library."""
    if not force and is_current():
        return LIB_PATH
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    srcs = source_files()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    procs = []
    objs = []
    extra = ["-Xptxas", "-v"] if verbose else []
    jobs = jobs or os.cpu_count() or 4
    pending = list(srcs)
    running: list[tuple[subprocess.Popen, Path]] = []
    logs: list[str] = []

    def reap(block: bool) -> None:
        for pr, src in list(running):
            if block:
                out, _ = pr.communicate()
            elif pr.poll() is None:
                continue
            else:
                out, _ = pr.communicate()
            running.remove((pr, src))
            text = out.decode(errors="replace")
            if verbose or pr.returncode != 0:
                logs.append(f"== {src.name}\n{text}")
            if pr.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{text}")

    while pending or running:
        while pending and len(running) < jobs:
            src = pending.pop(0)
            obj = obj_dir / (src.stem + ".o")
            objs.append(obj)
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            running.append((subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT), src))
        reap(block=not pending)
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs], "-cudart", "static"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout.decode(errors="replace"))
    STAMP_PATH.write_text(_digest())
    if verbose:
        sys.stdout.write("\n".join(logs) + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
