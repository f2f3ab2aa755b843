"""Re-shard a Hugging Face dataset into many files so every data-parallel rank / worker gets its own shards.

    python utils/reshard.py --dataset <name or path> [--name <config>] [--split train] --output <dir> [--num_shards 1024]

Datasets, not checkpoints: checkpoints are world-size independent already (utils/reshard.py:8-29 of the reference).
"""
import argparse

from datasets import load_dataset


def reshard(dataset: str, output: str, name: str = None, split: str = "train", num_shards: int = 1024) -> None:
    ds = load_dataset(dataset, name=name, split=split)
    ds.save_to_disk(output, num_shards=num_shards)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--name", default=None)
    ap.add_argument("--split", default="train")
    ap.add_argument("--output", required=True)
    ap.add_argument("--num_shards", type=int, default=1024)
    a = ap.parse_args()
    reshard(a.dataset, a.output, a.name, a.split, a.num_shards)
