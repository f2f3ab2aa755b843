"""Input pipeline: token streams -> fixed-length rows -> (optionally packed, varlen) batches.

Behavioural contract of the reference (flame/data.py:24-756):

* ``OnlineTokenizedIterableDataset``: the dataset is sharded by data-parallel rank, documents are tokenized
  64 at a time into one running token list, and fixed ``seq_len`` rows are emitted; the state (dataset position
  + left-over tokens) is checkpointable.
* ``BufferShuffledIterableDataset``: the same with a shuffle buffer of rows and a checkpointable RNG.
* ``DataCollatorForLanguageModeling``: non-varlen -> stack / pad (pad labels become -100); varlen -> batch size 1,
  ``cu_seqlens`` from BOS positions if the tokenizer has a BOS token, else from the positions after EOS tokens,
  then documents longer than ``context_len`` are split; labels are a plain copy (no masking across documents).
* ``ParallelAwareDataLoader``: state stored per data-parallel rank as ``{"rank_<k>": bytes}``.

Added here: ``SyntheticTokenDataset`` (documents of uniform random length joined by EOS, uniform tokens), used by
the benchmarks and by runs without network access, selected with ``--training.dataset synthetic``.
"""
from __future__ import annotations

import pickle
from typing import Any, Dict, Iterable, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, IterableDataset


# ----------------------------------------------------------------------------------------------------
# datasets
# ----------------------------------------------------------------------------------------------------
class SyntheticTokenDataset(IterableDataset):
    """Endless rows of ``seq_len`` tokens: documents with lengths uniform in [min_doc, max_doc] (EOS included),
    tokens uniform in [3, vocab_size), every document ends with ``eos_token_id``.  Deterministic in
    ``(seed, rank)`` and resumable."""

    def __init__(self, seq_len: int, vocab_size: int = 32000, min_doc: int = 64, max_doc: int = 4096,
                 eos_token_id: int = 2, bos_token_id: Optional[int] = None, seed: int = 42, rank: int = 0,
                 world_size: int = 1) -> None:
        self.seq_len, self.vocab_size = seq_len, vocab_size
        self.min_doc, self.max_doc = min_doc, max_doc
        self.eos, self.bos = eos_token_id, bos_token_id
        self.seed, self.rank, self.world_size = seed, rank, world_size
        self.rows_emitted = 0
        self._rng = np.random.default_rng([seed, rank])
        self._left: np.ndarray = np.empty(0, dtype=np.int64)

    def _document(self) -> np.ndarray:
        n = int(self._rng.integers(self.min_doc, self.max_doc + 1))
        doc = self._rng.integers(3, self.vocab_size, size=n, dtype=np.int64)
        doc[-1] = self.eos
        if self.bos is not None:
            doc[0] = self.bos
        return doc

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        while True:
            parts = [self._left]
            have = self._left.size
            while have < self.seq_len:
                d = self._document()
                parts.append(d)
                have += d.size
            buf = np.concatenate(parts)
            row, self._left = buf[: self.seq_len], buf[self.seq_len:]
            self.rows_emitted += 1
            yield {"input_ids": torch.from_numpy(row.copy())}

    def state_dict(self) -> Dict[str, Any]:
        return {"rows": self.rows_emitted, "rng": self._rng.bit_generator.state, "left": self._left.copy()}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.rows_emitted = sd["rows"]
        self._rng.bit_generator.state = sd["rng"]
        self._left = sd["left"]


class OnlineTokenizedIterableDataset(IterableDataset):
    """Tokenizes a (HF or any iterable-of-dicts) text dataset on the fly and yields ``seq_len`` token rows."""

    def __init__(self, dataset: Any, tokenizer: Any, seq_len: int = 2048, rank: int = 0, world_size: int = 1,
                 text_key: str = "text", docs_per_batch: int = 64) -> None:
        self.dataset, self.tokenizer, self.seq_len = dataset, tokenizer, seq_len
        self.rank, self.world_size, self.text_key, self.docs_per_batch = rank, world_size, text_key, docs_per_batch
        self.data = dataset.shard(world_size, rank) if hasattr(dataset, "shard") and world_size > 1 else dataset
        self.tokens: List[int] = []
        self.docs_consumed = 0
        self._resume_skip = 0

    def _token_batches(self) -> Iterator[List[int]]:
        batch: List[str] = []
        it = iter(self.data)
        skipped = 0
        for sample in it:
            if skipped < self._resume_skip and not hasattr(self.data, "load_state_dict"):
                skipped += 1
                continue
            text = sample[self.text_key] if isinstance(sample, dict) else sample
            batch.append(text)
            if len(batch) == self.docs_per_batch:
                yield from self._encode(batch)
                batch = []
        if batch:
            yield from self._encode(batch)

    def _encode(self, texts: List[str]) -> Iterator[List[int]]:
        enc = self.tokenizer(texts, return_attention_mask=False)["input_ids"]
        for ids in enc:
            self.docs_consumed += 1
            yield ids

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        while len(self.tokens) >= self.seq_len:
            row, self.tokens = self.tokens[: self.seq_len], self.tokens[self.seq_len:]
            yield {"input_ids": torch.tensor(row, dtype=torch.long)}
        for ids in self._token_batches():
            self.tokens.extend(ids)
            while len(self.tokens) >= self.seq_len:
                row, self.tokens = self.tokens[: self.seq_len], self.tokens[self.seq_len:]
                yield {"input_ids": torch.tensor(row, dtype=torch.long)}

    def state_dict(self) -> Dict[str, Any]:
        sd: Dict[str, Any] = {"tokens": list(self.tokens), "docs": self.docs_consumed}
        if hasattr(self.data, "state_dict"):
            sd["data"] = self.data.state_dict()
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.tokens = list(sd["tokens"])
        self.docs_consumed = sd.get("docs", 0)
        if "data" in sd and hasattr(self.data, "load_state_dict"):
            self.data.load_state_dict(sd["data"])
        else:
            self._resume_skip = self.docs_consumed


class BufferShuffledIterableDataset(IterableDataset):
    """Rows pass through a shuffle buffer of ``buffer_size`` rows; the RNG state is part of the checkpoint."""

    def __init__(self, source: IterableDataset, buffer_size: int = 1024, seed: int = 42) -> None:
        self.source, self.buffer_size = source, buffer_size
        self.rng = np.random.default_rng(seed)
        self.buffer: List[Dict[str, torch.Tensor]] = []

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        for row in self.source:
            if len(self.buffer) < self.buffer_size:
                self.buffer.append(row)
                continue
            i = int(self.rng.integers(0, self.buffer_size))
            out, self.buffer[i] = self.buffer[i], row
            yield out
        order = self.rng.permutation(len(self.buffer))
        for i in order:
            yield self.buffer[int(i)]
        self.buffer = []

    def state_dict(self) -> Dict[str, Any]:
        sd = {"rng": self.rng.bit_generator.state, "buffer": [r["input_ids"].clone() for r in self.buffer]}
        if hasattr(self.source, "state_dict"):
            sd["source"] = self.source.state_dict()
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.rng.bit_generator.state = sd["rng"]
        self.buffer = [{"input_ids": t} for t in sd["buffer"]]
        if "source" in sd and hasattr(self.source, "load_state_dict"):
            self.source.load_state_dict(sd["source"])


# ----------------------------------------------------------------------------------------------------
# collator
# ----------------------------------------------------------------------------------------------------
class DataCollatorForLanguageModeling:
    def __init__(self, tokenizer: Any, context_len: Optional[int] = None, varlen: bool = False) -> None:
        self.tokenizer, self.context_len, self.varlen = tokenizer, context_len, varlen
        if varlen and getattr(tokenizer, "bos_token_id", None) is None and getattr(tokenizer, "eos_token_id", None) is None:
            raise ValueError("varlen batches need a tokenizer with a BOS or an EOS token to find document boundaries")

    def __call__(self, examples: List[Any]) -> Dict[str, torch.Tensor]:
        rows = [e["input_ids"] if isinstance(e, dict) else e for e in examples]
        rows = [r if isinstance(r, torch.Tensor) else torch.tensor(r, dtype=torch.long) for r in rows]
        if not self.varlen:
            return self._dense(rows)
        if len(rows) > 1:
            raise ValueError("The batch size must be 1 for inputs with variable lengths (varlen=True).")
        ids = rows[0].reshape(1, -1)
        if isinstance(examples[0], dict) and "cu_seqlens" in examples[0]:
            cu = examples[0]["cu_seqlens"].to(torch.int32).reshape(-1)
        else:
            cu = self.boundaries(ids[0])
        cu = self.split_long(cu, ids.shape[1])
        return {"input_ids": ids, "labels": ids.clone(), "cu_seqlens": cu}

    def _dense(self, rows: List[torch.Tensor]) -> Dict[str, torch.Tensor]:
        L = max(r.numel() for r in rows)
        if all(r.numel() == L for r in rows):
            ids = torch.stack(rows)
            labels = ids.clone()
        else:
            pad = getattr(self.tokenizer, "pad_token_id", None)
            if pad is None:
                raise ValueError("rows of different length need a tokenizer with a pad token")
            ids = torch.full((len(rows), L), pad, dtype=torch.long)
            labels = torch.full((len(rows), L), -100, dtype=torch.long)
            for i, r in enumerate(rows):
                ids[i, : r.numel()] = r
                labels[i, : r.numel()] = r
        pad = getattr(self.tokenizer, "pad_token_id", None)
        if pad is not None:
            labels[ids == pad] = -100
        return {"input_ids": ids, "labels": labels}

    def boundaries(self, row: torch.Tensor) -> torch.Tensor:
        """Document starts: BOS positions when the tokenizer defines BOS, otherwise the positions after EOS."""
        n = row.numel()
        bos = getattr(self.tokenizer, "bos_token_id", None)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if bos is not None:
            starts = torch.nonzero(row == bos).flatten()
            pieces = []
            if n == 0 or row[0] != bos:
                pieces.append(torch.zeros(1, dtype=torch.long))
            pieces += [starts, torch.tensor([n])]
        else:
            ends = torch.nonzero(row == eos).flatten() + 1
            pieces = [torch.zeros(1, dtype=torch.long), ends]
            if n == 0 or row[-1] != eos:
                pieces.append(torch.tensor([n]))
        cu = torch.cat(pieces).to(torch.int32)
        if cu.numel() < 2 or cu[0] != 0 or cu[-1] != n or not bool((cu[1:] >= cu[:-1]).all()):
            raise ValueError(f"invalid document boundaries {cu.tolist()} for a row of {n} tokens")
        return cu

    def split_long(self, cu: torch.Tensor, n: int) -> torch.Tensor:
        """Cut documents longer than ``context_len``; drops empty documents and duplicate boundaries."""
        if self.context_len is None:
            return torch.unique(cu)
        pts = [torch.arange(int(a), int(b), self.context_len) for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()) if a < b]
        if not pts:
            return torch.tensor([0, 0], dtype=torch.int32)
        return torch.unique(torch.cat(pts + [torch.tensor([n])])).to(torch.int32)


# ----------------------------------------------------------------------------------------------------
# loader
# ----------------------------------------------------------------------------------------------------
class ParallelAwareDataLoader:
    """Iterable of collated batches with a per-data-parallel-rank checkpoint state.

    The dataset runs in the trainer process by default (``num_workers=0``): tokenisation of 64-document batches
    costs far less than a training step on one B200 and keeps the state exact.  ``num_workers > 0`` delegates to
    ``torchdata``'s ``StatefulDataLoader``."""

    def __init__(self, rank: int, dataset: IterableDataset, batch_size: int, collate_fn, num_workers: int = 0,
                 pin_memory: bool = False, persistent_workers: bool = False, prefetch_factor: Optional[int] = 2,
                 snapshot_every_n_steps: Optional[int] = 1) -> None:
        self.rank, self.dataset, self.batch_size, self.collate_fn = rank, dataset, batch_size, collate_fn
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self._rank_id = f"rank_{rank}"
        self._inner = None
        if num_workers > 0:
            from torchdata.stateful_dataloader import StatefulDataLoader
            self._inner = StatefulDataLoader(dataset, batch_size=batch_size, collate_fn=collate_fn,
                                             num_workers=num_workers, pin_memory=self.pin_memory,
                                             persistent_workers=persistent_workers,
                                             prefetch_factor=prefetch_factor,
                                             snapshot_every_n_steps=snapshot_every_n_steps)

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        if self._inner is not None:
            yield from self._inner
            return
        rows: List[Any] = []
        for row in self.dataset:
            rows.append(row)
            if len(rows) == self.batch_size:
                batch = self.collate_fn(rows)
                if self.pin_memory:
                    batch = {k: v.pin_memory() for k, v in batch.items()}
                yield batch
                rows = []

    def state_dict(self) -> Dict[str, Any]:
        inner = self._inner.state_dict() if self._inner is not None else (
            self.dataset.state_dict() if hasattr(self.dataset, "state_dict") else {})
        return {self._rank_id: pickle.dumps(inner)}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        if not state_dict:
            return
        if self._rank_id not in state_dict:
            return  # resumed with a different data-parallel degree: this rank starts its shard from the beginning
        inner = pickle.loads(state_dict[self._rank_id])
        if self._inner is not None:
            self._inner.load_state_dict(inner)
        elif hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(inner)


class SimpleTokenizer:
    """Stand-in tokenizer for synthetic data and tests: carries the special ids and a vocab size."""

    def __init__(self, vocab_size: int = 32000, bos_token_id: Optional[int] = None, eos_token_id: Optional[int] = 2,
                 pad_token_id: Optional[int] = None) -> None:
        self.vocab_size, self.bos_token_id, self.eos_token_id, self.pad_token_id = vocab_size, bos_token_id, eos_token_id, pad_token_id

    def __call__(self, texts, return_attention_mask: bool = False):
        out = []
        for t in texts:
            ids = [3 + (ord(c) % (self.vocab_size - 3)) for c in t]
            if self.bos_token_id is not None:
                ids = [self.bos_token_id] + ids
            if self.eos_token_id is not None:
                ids = ids + [self.eos_token_id]
            out.append(ids)
        return {"input_ids": out}

    def save_pretrained(self, path: str) -> None:
        import json
        import os
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "simple_tokenizer.json"), "w") as f:
            json.dump(self.__dict__, f)

    def __repr__(self) -> str:
        return f"SimpleTokenizer({self.__dict__})"


def build_tokenizer(path: str, vocab_size: int = 32000):
    """``synthetic`` (or a missing path) gives the stand-in tokenizer; anything else goes to ``AutoTokenizer``."""
    import os
    if path in ("synthetic", "", None) or (not os.path.exists(path) and "/" not in str(path)):
        return SimpleTokenizer(vocab_size=vocab_size)
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path, trust_remote_code=True, model_max_length=int(1e10))
    except Exception as e:  # no network / not a tokenizer directory
        raise RuntimeError(f"cannot load tokenizer {path!r}: {e}") from e


def build_dataset(dataset: str, dataset_name: Optional[str] = None, dataset_split: Optional[str] = None,
                  data_dir: Optional[str] = None, data_files: Optional[str] = None, data_probs: Optional[str] = None,
                  streaming: bool = False, dp_degree: int = 1, num_workers: int = 0, seed: int = 42, **kw) -> Any:
    """A single dataset or a comma-separated mixture (``data_probs``) from HF ``datasets``; map-style datasets are
    shuffled and converted to iterable form with ``dp_degree * max(num_workers, 1)`` shards
    (flame/data.py:545-727).  ``synthetic`` returns a marker that ``build_dataloader`` turns into a
    ``SyntheticTokenDataset``."""
    if dataset == "synthetic":
        return "synthetic"
    from datasets import interleave_datasets, load_dataset, load_from_disk
    import os
    names = dataset.split(",")

    def pick(val: Optional[str], i: int) -> Optional[str]:
        if val is None:
            return None
        parts = val.split(",")
        return parts[i] if len(parts) > 1 else parts[0]

    built = []
    for i, name in enumerate(names):
        split = pick(dataset_split, i) or "train"
        if os.path.isdir(name) and os.path.exists(os.path.join(name, "dataset_info.json")):
            ds = load_from_disk(name)
        else:
            ds = load_dataset(path=name, name=pick(dataset_name, i), split=split, data_dir=pick(data_dir, i),
                              data_files=pick(data_files, i), streaming=streaming, trust_remote_code=True)
        shards = dp_degree * max(num_workers, 1)
        if not streaming and hasattr(ds, "to_iterable_dataset"):
            ds = ds.shuffle(seed=seed).to_iterable_dataset(num_shards=shards)
        elif hasattr(ds, "shuffle"):
            ds = ds.shuffle(seed=seed)
        built.append(ds)
    if len(built) == 1:
        return built[0]
    probs = [float(p) for p in data_probs.split(",")] if data_probs else None
    if probs is None or len(probs) != len(built):
        raise ValueError("a dataset mixture needs one probability per dataset in --training.data_probs")
    return interleave_datasets(built, probabilities=probs, stopping_strategy="all_exhausted", seed=seed)


def build_dataloader(dataset: Any, tokenizer: Any, rank: int, world_size: int, batch_size: int, seq_len: int,
                     context_len: Optional[int] = None, varlen: bool = False, num_workers: int = 0,
                     pin_memory: bool = False, persistent_workers: bool = False,
                     snapshot_every_n_steps: Optional[int] = 1, seed: int = 42, vocab_size: int = 32000,
                     synthetic_doc_range=(64, 4096)) -> ParallelAwareDataLoader:
    if isinstance(dataset, str) and dataset == "synthetic":
        ds: IterableDataset = SyntheticTokenDataset(
            seq_len, vocab_size=vocab_size, min_doc=synthetic_doc_range[0], max_doc=synthetic_doc_range[1],
            eos_token_id=getattr(tokenizer, "eos_token_id", 2) or 2, bos_token_id=None, seed=seed, rank=rank,
            world_size=world_size)
        num_workers = 0
    else:
        ds = OnlineTokenizedIterableDataset(dataset, tokenizer, seq_len, rank, world_size)
    collate = DataCollatorForLanguageModeling(tokenizer, context_len=context_len, varlen=varlen)
    return ParallelAwareDataLoader(rank, ds, batch_size, collate, num_workers=num_workers, pin_memory=pin_memory,
                                   persistent_workers=persistent_workers, snapshot_every_n_steps=snapshot_every_n_steps)
