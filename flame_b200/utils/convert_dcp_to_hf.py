"""Export a training checkpoint (torch-DCP) as a Hugging Face style model directory.

    python -m flame_b200.utils.convert_dcp_to_hf --path exp/run --step 20480 --config configs/transformer_340M.json \
        [--tokenizer <dir>]

Reads ``<path>/checkpoint/step-<N>``, takes the ``model`` sub-tree and writes ``config.json`` + ``model.safetensors``
(+ tokenizer files) into ``<path>``; same contract as flame/utils/convert_dcp_to_hf.py:20-65.
"""
from __future__ import annotations

import argparse
import io
import os
import tempfile
from datetime import timedelta

import torch
import torch.serialization
from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

from ..components.metrics import init_logger, logger
from ..models import ModelConfig, build_model


@torch.inference_mode()
def save_pretrained(path: str, step: int, config: str, tokenizer: str | None = None, dtype: str = "float32") -> None:
    cfg = ModelConfig.from_pretrained(config)
    ckpt = os.path.join(path, "checkpoint", f"step-{step}")
    with tempfile.TemporaryDirectory() as tmp:
        flat = os.path.join(tmp, "checkpoint.pt")
        logger.info(f"Reading the distributed checkpoint {ckpt}")
        dcp_to_torch_save(ckpt, flat)
        torch.serialization.add_safe_globals([timedelta, io.BytesIO])
        state = torch.load(flat, map_location="cpu", weights_only=False)
    sd = state["model"] if "model" in state else state
    model = build_model(cfg, device="cpu", dtype=torch.float32, init=False)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"checkpoint does not match the config: missing={missing[:4]} unexpected={unexpected[:4]}")
    td = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[dtype]
    model.save_pretrained(path, dtype=td)
    if tokenizer and os.path.isdir(tokenizer):
        from transformers import AutoTokenizer
        AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=True).save_pretrained(path)
    logger.info(f"Saved the model to {path}")


def main() -> None:
    init_logger()
    ap = argparse.ArgumentParser("Convert a DCP checkpoint to a HF model directory")
    ap.add_argument("--path", required=True)
    ap.add_argument("--step", type=int, required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--dtype", default="float32")
    a = ap.parse_args()
    save_pretrained(a.path, a.step, a.config, a.tokenizer, a.dtype)


if __name__ == "__main__":
    main()
