"""Turn a Hugging Face style model directory into a step-0 training checkpoint.

    python -m flame_b200.utils.convert_hf_to_dcp --model <hf dir> --checkpoint exp/run/checkpoint/step-0

Writes ``{"model": state_dict}`` with torch-DCP (flame/utils/convert_hf_to_dcp.py:15-34); a trainer started with
``--checkpoint.load_step 0`` (or with that folder as ``initial_load_path``) picks the weights up.
"""
from __future__ import annotations

import argparse
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp

from ..components.metrics import init_logger, logger
from ..models import CausalLM


@torch.inference_mode()
def convert_hf_weights(model: str, checkpoint: str) -> None:
    logger.info(f"Loading model from {model}")
    m = CausalLM.from_pretrained(model)
    sd = {k: v.float().contiguous() for k, v in m.state_dict().items()}
    Path(checkpoint).mkdir(parents=True, exist_ok=True)
    dcp.save({"model": sd}, storage_writer=dcp.filesystem.FileSystemWriter(checkpoint, thread_count=8), no_dist=True)
    logger.info(f"Wrote DCP checkpoint to {checkpoint}")


def main() -> None:
    init_logger()
    ap = argparse.ArgumentParser("Convert HF weights to a DCP checkpoint")
    ap.add_argument("--model", required=True)
    ap.add_argument("--checkpoint", required=True)
    a = ap.parse_args()
    convert_hf_weights(a.model, a.checkpoint)


if __name__ == "__main__":
    main()
