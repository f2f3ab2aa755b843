"""Input pipeline: token streams -> fixed-length rows -> (optionally packed, varlen) batches.

Behavioural contract of the reference (flame/data.py:24-756):

* ``OnlineTokenizedIterableDataset``: the dataset is sharded by data-parallel rank, documents are tokenized
  64 at a time into one running token list, and fixed ``seq_len`` rows are emitted; the state (dataset position
  + left-over tokens) is checkpointable.
* ``BufferShuffledIterableDataset``: the same with a shuffle buffer of rows and a checkpointable RNG.
* ``ShuffledExampleStream`` / ``shuffle``: resumable example-level shuffle of a streaming dataset; ``build_dataset``
  uses it for streaming datasets and falls back to a map-style load when the stream has too few shards.
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


def _sample_text(sample: Any) -> str:
    """The document text of one dataset sample: ``text``, else ``content`` (flame/data.py:188-194)."""
    if isinstance(sample, str):
        return sample
    for key in ("text", "content"):
        if sample.get(key, None) is not None:
            return sample[key]
    raise ValueError(f"No 'text' or 'content' field found in sample:\n{sample}")


class OnlineTokenizedIterableDataset(IterableDataset):
    """Tokenizes a (HF or any iterable-of-dicts) text dataset on the fly and yields ``seq_len`` token rows, forever.

    Documents are read ``docs_per_batch`` at a time and tokenized in one call.  The source position is recorded PER
    DOCUMENT while the batch is read, and the checkpoint keeps the position that belongs to the last document whose
    tokens were taken into the running token list, so a resume continues with exactly the next document: nothing of
    the read-ahead batch is lost (flame/data.py:171-210).  When the source runs out it is started again (the
    reference's endless epoch loop), so a dataset shorter than the run never ends it.  A source with
    ``state_dict / load_state_dict`` (HF iterable datasets, ``ShuffledExampleStream``) is resumed through them;
    any other iterable is resumed by counting documents inside the current pass."""

    def __init__(self, dataset: Any, tokenizer: Any, seq_len: int = 2048, rank: int = 0, world_size: int = 1,
                 docs_per_batch: int = 64) -> None:
        self.dataset, self.tokenizer, self.seq_len = dataset, tokenizer, seq_len
        self.rank, self.world_size, self.docs_per_batch = rank, world_size, docs_per_batch
        if hasattr(dataset, "shard") and world_size > 1:
            self.data = dataset.shard(world_size, rank)
        elif world_size > 1 and isinstance(dataset, (list, tuple)):
            self.data = dataset[rank::world_size]
        else:
            self.data = dataset
        self._stateful = hasattr(self.data, "state_dict") and hasattr(self.data, "load_state_dict")
        self.tokens: List[int] = []
        self.states: Any = None   # source position after the last consumed document
        self.epoch = 0            # completed passes over the source
        self.docs_in_pass = 0     # documents consumed in the current pass (position of a stateless source)

    def _documents(self) -> Iterator[List[int]]:
        """Token lists of the source's documents from the current position to the end of this pass."""
        if self._stateful:
            if self.states is not None:
                self.data.load_state_dict(self.states)
            source = iter(self.data)
        else:
            source = iter(self.data)
            for _ in range(self.docs_in_pass):
                if next(source, None) is None:
                    break
        texts: List[str] = []
        marks: List[Any] = []

        def flush() -> Iterator[List[int]]:
            enc = self.tokenizer(texts, return_attention_mask=False)["input_ids"]
            for mark, ids in zip(marks, enc):
                self.states = mark
                self.docs_in_pass += 1
                yield ids

        for sample in source:
            texts.append(_sample_text(sample))
            marks.append(self.data.state_dict() if self._stateful else None)
            if len(texts) == self.docs_per_batch:
                yield from flush()
                texts, marks = [], []
        if texts:
            yield from flush()

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        while True:
            got_any = False
            for ids in self._documents():
                got_any = True
                self.tokens += ids
                while len(self.tokens) >= self.seq_len:
                    row, self.tokens = self.tokens[: self.seq_len], self.tokens[self.seq_len:]
                    yield {"input_ids": torch.tensor(row, dtype=torch.long)}
            if not got_any and self.docs_in_pass == 0:
                raise ValueError("the dataset shard of this rank is empty")
            # the pass is over: start the source again
            self.epoch += 1
            self.docs_in_pass = 0
            self.states = None
            if self._stateful and hasattr(self.data, "set_epoch"):
                self.data.set_epoch(self.epoch)

    def state_dict(self) -> Dict[str, Any]:
        import copy
        return {"states": copy.deepcopy(self.states), "tokens": list(self.tokens), "epoch": self.epoch,
                "docs_in_pass": self.docs_in_pass}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        import copy
        self.states = copy.deepcopy(sd.get("states"))
        self.tokens = list(sd["tokens"])
        self.epoch = sd.get("epoch", 0)
        self.docs_in_pass = sd.get("docs_in_pass", sd.get("docs", 0))
        if self._stateful and self.epoch and hasattr(self.data, "set_epoch"):
            self.data.set_epoch(self.epoch)


class ShuffledExampleStream:
    """Resumable example-level shuffle of a streaming dataset (the role of the reference's
    ``BufferShuffledExamplesIterable`` + ``shuffle``, flame/data.py:213-308).

    Examples pass through a reservoir of ``buffer_size`` slots: once it is full, every incoming example replaces a
    uniformly drawn slot and the evicted example is emitted; when the source ends, what is left is emitted in a random
    order.  The whole state - the reservoir's contents, the generator's state, the source position (its own
    ``state_dict`` when it has one, else the number of examples drawn) and how much of the final drain was emitted - is
    checkpointable, so a resumed stream continues with the same examples in the same order.  ``shard`` forwards to the
    source, so it composes with ``OnlineTokenizedIterableDataset``."""

    def __init__(self, source: Any, seed: int = 42, buffer_size: int = 1024) -> None:
        self.source, self.seed, self.buffer_size = source, seed, buffer_size
        self._stateful = hasattr(source, "state_dict") and hasattr(source, "load_state_dict")
        self._reset()

    def _reset(self) -> None:
        self.rng = np.random.default_rng(self.seed)
        self.buffer: List[Any] = []
        self.drawn = 0               # examples taken from the source so far
        self.source_state: Any = None
        self.drain_order: Optional[List[int]] = None
        self.drain_pos = 0

    @property
    def num_shards(self) -> int:
        return int(getattr(self.source, "num_shards", getattr(self.source, "n_shards", 1)))

    n_shards = num_shards

    @property
    def column_names(self):
        return getattr(self.source, "column_names", None)

    def shard(self, num_shards: int, index: int) -> "ShuffledExampleStream":
        if hasattr(self.source, "shard"):
            src = self.source.shard(num_shards, index)
        else:
            src = list(self.source)[index::num_shards]
        return ShuffledExampleStream(src, seed=self.seed, buffer_size=self.buffer_size)

    def set_epoch(self, epoch: int) -> None:
        """A new pass over the source: fresh reservoir, generator seeded by (seed, epoch)."""
        self._reset()
        self.rng = np.random.default_rng([self.seed, epoch])
        if hasattr(self.source, "set_epoch"):
            self.source.set_epoch(epoch)

    def __iter__(self) -> Iterator[Any]:
        if self.drain_order is None:
            if self._stateful:
                if self.source_state is not None:
                    self.source.load_state_dict(self.source_state)
                it = iter(self.source)
            else:
                it = iter(self.source)
                for _ in range(self.drawn):
                    if next(it, None) is None:
                        break
            for x in it:
                self.drawn += 1
                if len(self.buffer) < self.buffer_size:
                    self.buffer.append(x)
                    if self._stateful:
                        self.source_state = self.source.state_dict()
                    continue
                i = int(self.rng.integers(0, self.buffer_size))
                out, self.buffer[i] = self.buffer[i], x
                if self._stateful:
                    self.source_state = self.source.state_dict()
                yield out
            self.drain_order = [int(i) for i in self.rng.permutation(len(self.buffer))]
            self.drain_pos = 0
        while self.drain_pos < len(self.drain_order):
            i = self.drain_order[self.drain_pos]
            self.drain_pos += 1
            yield self.buffer[i]

    def state_dict(self) -> Dict[str, Any]:
        import copy
        return {"rng": copy.deepcopy(self.rng.bit_generator.state), "buffer": list(self.buffer), "drawn": self.drawn,
                "source": copy.deepcopy(self.source_state), "drain_order": None if self.drain_order is None else list(self.drain_order),
                "drain_pos": self.drain_pos}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.rng = np.random.default_rng(self.seed)
        self.rng.bit_generator.state = sd["rng"]
        self.buffer = list(sd["buffer"])
        self.drawn = sd["drawn"]
        self.source_state = sd["source"]
        self.drain_order = None if sd["drain_order"] is None else list(sd["drain_order"])
        self.drain_pos = sd["drain_pos"]


def shuffle(dataset: Any, seed: int = 42, buffer_size: int = 1024) -> ShuffledExampleStream:
    """Resumable buffer shuffle of a streaming dataset (flame/data.py:291-308)."""
    return ShuffledExampleStream(dataset, seed=seed, buffer_size=buffer_size)


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
                  streaming: bool = False, dp_degree: int = 1, num_workers: int = 0, seed: int = 42,
                  loader=None, **kw) -> Any:
    """A single dataset or a comma-separated mixture (``data_probs``) from HF ``datasets`` (flame/data.py:545-727).

    * map-style: shuffled with ``seed`` and converted to iterable form with ``dp_degree * num_workers`` shards;
    * streaming with enough shards for ``dp_degree x num_workers`` readers: resumable buffer shuffle (``shuffle``;
      1024 examples, ``max(128, 1024 // n)`` per member of a mixture of n);
    * streaming with too few shards: a warning, then the dataset is loaded map-style and resharded instead;
    * mixtures keep only the ``text`` (else ``content``) column and are interleaved until all are exhausted.

    ``synthetic`` returns a marker that ``build_dataloader`` turns into a ``SyntheticTokenDataset``.  ``loader`` replaces
    ``datasets.load_dataset`` (tests)."""
    if dataset == "synthetic":
        return "synthetic"
    import os
    from .components.metrics import logger
    if loader is None:
        from datasets import load_dataset, load_from_disk

        def loader(path, **kwargs):
            if os.path.isdir(path) and os.path.exists(os.path.join(path, "dataset_info.json")):
                return load_from_disk(path)
            return load_dataset(path=path, trust_remote_code=True, **kwargs)

    names = dataset.split(",")
    n = len(names)
    min_shards = dp_degree * max(num_workers, 1) if dp_degree else None

    def column(val: Optional[str], what: str, default=None) -> List[Optional[str]]:
        if val is None:
            return [default] * n
        parts = [p or default for p in val.split(",")] if n > 1 else [val]
        if len(parts) != n:
            raise ValueError(f"The number of {what} must match the number of datasets")
        return parts

    ds_names, splits = column(dataset_name, "dataset names"), column(dataset_split, "dataset splits", "train")
    dirs, files = column(data_dir, "data dirs"), column(data_files, "data files")
    probs = None
    if n > 1:
        if data_probs is None:
            raise ValueError("Data sampling probabilities are required if using multiple datasets")
        probs = [float(p) for p in str(data_probs).split(",")]
        if len(probs) != n:
            raise ValueError("The number of data probabilities must match the number of datasets")

    def load_one(i: int, stream: bool):
        return loader(names[i], name=ds_names[i], split=splits[i], data_dir=dirs[i], data_files=files[i],
                      streaming=stream, **({"num_proc": num_workers} if (not stream and num_workers > 0) else {}))

    def to_shards(ds):
        if seed is not None and hasattr(ds, "shuffle"):
            ds = ds.shuffle(seed=seed)
        if min_shards is not None and hasattr(ds, "to_iterable_dataset"):
            ds = ds.to_iterable_dataset(num_shards=min_shards)
        return ds

    built = []
    for i in range(n):
        ds = load_one(i, streaming)
        if not streaming:
            ds = to_shards(ds)
        else:
            have = int(getattr(ds, "num_shards", getattr(ds, "n_shards", 1)))
            if min_shards is not None and have < min_shards:
                logger.warning(f"Dataset {names[i]} has insufficient shards ({have}). Need {min_shards} shards minimum for "
                               f"{dp_degree} data parallel workers x {num_workers} dataloader workers. Disabling the "
                               f"streaming mode and resharding dataset to {min_shards} shards.")
                ds = to_shards(load_one(i, False))
            elif seed is not None:
                ds = shuffle(ds, seed=seed, buffer_size=1024 if n == 1 else max(128, 1024 // n))
        if n > 1:
            cols = getattr(ds, "column_names", None)
            if cols is not None and hasattr(ds, "select_columns"):
                if "text" in cols:
                    ds = ds.select_columns("text")
                elif "content" in cols:
                    ds = ds.select_columns("content")
                else:
                    raise ValueError(f"Subset {names[i]} has no 'text' or 'content' column")
        built.append(ds)
    if n == 1:
        return built[0]
    if all(hasattr(d, "_ex_iterable") or hasattr(d, "features") for d in built):
        from datasets import interleave_datasets
        return interleave_datasets(built, probabilities=probs, stopping_strategy="all_exhausted", seed=seed)
    return InterleavedStreams(built, probs, seed=seed)


class InterleavedStreams:
    """Draws the next example from member ``i`` with probability ``probs[i]`` until every member was exhausted once
    (an exhausted member starts again, HF's ``all_exhausted`` strategy), for members that are not HF datasets (for
    example ``ShuffledExampleStream``).  Resumable through the members' states and the generator's state."""

    def __init__(self, members: List[Any], probs: List[float], seed: int = 42) -> None:
        self.members, self.seed = members, seed
        p = np.asarray(probs, dtype=np.float64)
        self.probs = p / p.sum()
        self.rng = np.random.default_rng(seed)
        self._pending_state: Optional[Dict[str, Any]] = None

    def shard(self, num_shards: int, index: int) -> "InterleavedStreams":
        return InterleavedStreams([m.shard(num_shards, index) if hasattr(m, "shard") else list(m)[index::num_shards]
                                   for m in self.members], list(self.probs), seed=self.seed)

    def __iter__(self) -> Iterator[Any]:
        iters = [iter(m) for m in self.members]
        done = [False] * len(iters)
        while not all(done):
            i = int(self.rng.choice(len(iters), p=self.probs))
            x = next(iters[i], None)
            if x is None:
                done[i] = True
                if all(done):
                    return
                if hasattr(self.members[i], "set_epoch"):
                    self.members[i].set_epoch(1)
                iters[i] = iter(self.members[i])
                x = next(iters[i], None)
                if x is None:
                    continue
            yield x

    def state_dict(self) -> Dict[str, Any]:
        import copy
        return {"rng": copy.deepcopy(self.rng.bit_generator.state),
                "members": [m.state_dict() if hasattr(m, "state_dict") else None for m in self.members]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.rng.bit_generator.state = sd["rng"]
        for m, st in zip(self.members, sd["members"]):
            if st is not None and hasattr(m, "load_state_dict"):
                m.load_state_dict(st)


def build_dataloader(dataset: Any, tokenizer: Any, rank: int, world_size: int, batch_size: int, seq_len: int,
                     context_len: Optional[int] = None, varlen: bool = False, num_workers: int = 0,
                     pin_memory: bool = False, persistent_workers: bool = False,
                     snapshot_every_n_steps: Optional[int] = 1, seed: int = 42, vocab_size: int = 32000,
                     synthetic_doc_range=(64, 4096), prefetch_factor: Optional[int] = 2) -> ParallelAwareDataLoader:
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
                                   persistent_workers=persistent_workers, snapshot_every_n_steps=snapshot_every_n_steps,
                                   prefetch_factor=prefetch_factor if num_workers > 0 else None)
