"""Offline tokenisation: ``dataset.map(tokenize)`` -> ``save_to_disk`` with ``input_ids`` and ``bits_per_token``.

    python -m flame_b200.utils.preprocess --dataset <name or path> --tokenizer <dir> --output <dir> [--num_proc 64]

Same output columns as flame/utils/preprocess.py:13-122 so pre-tokenised datasets interchange.
"""
from __future__ import annotations

import argparse
from typing import Any, Dict, List

from ..components.metrics import init_logger, logger


def tokenize(examples: Dict[str, List[Any]], tokenizer) -> Dict[str, List[Any]]:
    texts = examples["text"] if "text" in examples else examples["content"]
    ids = tokenizer(texts)["input_ids"]
    nbytes = [len(t.encode("utf-8")) for t in texts]
    bits = [8.0 * b / max(len(i), 1) for b, i in zip(nbytes, ids)]
    return {"input_ids": ids, "bits_per_token": bits}


def main() -> None:
    init_logger()
    ap = argparse.ArgumentParser("Tokenize a dataset once and store it on disk")
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--name", default=None)
    ap.add_argument("--split", default="train")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--num_proc", type=int, default=8)
    ap.add_argument("--batch_size", type=int, default=2048)
    a = ap.parse_args()
    from datasets import load_dataset
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.tokenizer, trust_remote_code=True)
    ds = load_dataset(a.dataset, name=a.name, split=a.split)
    ds = ds.map(lambda ex: tokenize(ex, tok), batched=True, batch_size=a.batch_size, num_proc=a.num_proc,
                remove_columns=ds.column_names, desc="tokenizing")
    ds.save_to_disk(a.output)
    logger.info(f"Saved {len(ds)} tokenised documents to {a.output}")


if __name__ == "__main__":
    main()
