"""Reference arm of ``bench.py``: runs the reference trainer installed under ``baseline/_ref`` on the benchmark recipe.

The install (``pip install --no-index --no-deps --target baseline/_ref``) succeeds, but the package does not import
on this image: it is written against an older torchtitan than the one installed (``FTParallelDims``,
``torchtitan.config_manager`` and several builder signatures are gone).  Until a compatibility layer for those
symbols exists the arm reports itself unavailable.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def probe() -> str:
    """Empty string when ``flame.train`` of the reference imports, else the reason."""
    if not os.path.isdir(os.path.join(REF, "flame")):
        return "reference is not installed under baseline/_ref"
    sys.path.insert(0, REF)
    try:
        import importlib
        importlib.import_module("flame.train")
        return ""
    except Exception as e:
        return f"reference does not import on this image: {type(e).__name__}: {str(e)[:160]}"
    finally:
        if REF in sys.path:
            sys.path.remove(REF)


def run(args, seq_len: int, context_len: int, model_json: str) -> dict:
    why = probe()
    if why:
        return {"impl": "reference", "unavailable": why}
    return {"impl": "reference", "unavailable": "reference imports but no runner is wired for it yet"}
