"""Input pipeline on CPU: tokenising dataset (endless, resumable per document), resumable streaming shuffle, the
too-few-shards fallback of ``build_dataset``, the collator's boundary rules and the per-rank loader state.
Behaviour under test is the reference's (flame/data.py:156-210, 213-308, 389-496, 501-542, 545-727)."""
import itertools

import pytest
import torch

from flame_b200.data import (DataCollatorForLanguageModeling, InterleavedStreams, OnlineTokenizedIterableDataset,
                             ParallelAwareDataLoader, ShuffledExampleStream, SimpleTokenizer, build_dataloader,
                             build_dataset, shuffle)


def _docs(n, key="text"):
    return [{key: "".join(chr(97 + (i * 7 + j) % 26) for j in range(5 + (i * 13) % 40))} for i in range(n)]


class StatefulList:
    """A source with HF's iterable-dataset state protocol: the state is the index of the next sample."""

    def __init__(self, items, num_shards=4):
        self.items, self.pos, self.num_shards = items, 0, num_shards
        self.column_names = list(items[0].keys()) if items and isinstance(items[0], dict) else None

    def shard(self, n, i):
        return StatefulList(self.items[i::n], self.num_shards)

    def __iter__(self):
        while self.pos < len(self.items):
            x = self.items[self.pos]
            self.pos += 1
            yield x
        self.pos = 0  # a fresh iterator starts over, like an HF dataset whose state was consumed

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = sd["pos"]


def _rows(ds, n):
    return [r["input_ids"].tolist() for r in itertools.islice(iter(ds), n)]


@pytest.mark.parametrize("stateful", [False, True])
def test_resume_inside_a_tokenizer_batch_loses_no_document(stateful):
    tok = SimpleTokenizer(vocab_size=500)
    make = (lambda: StatefulList(_docs(200))) if stateful else (lambda: _docs(200))
    full = _rows(OnlineTokenizedIterableDataset(make(), tok, seq_len=32, docs_per_batch=16), 40)
    a = OnlineTokenizedIterableDataset(make(), tok, seq_len=32, docs_per_batch=16)
    it = iter(a)
    head = [next(it)["input_ids"].tolist() for _ in range(7)]  # stops in the middle of a 16-document batch
    sd = a.state_dict()
    b = OnlineTokenizedIterableDataset(make(), tok, seq_len=32, docs_per_batch=16)
    b.load_state_dict(sd)
    tail = _rows(b, 33)
    assert head + tail == full


def test_short_dataset_repeats_instead_of_ending_the_run():
    tok = SimpleTokenizer(vocab_size=500)
    ds = OnlineTokenizedIterableDataset(_docs(5), tok, seq_len=64)
    rows = _rows(ds, 30)  # far more tokens than one pass holds
    assert len(rows) == 30 and ds.epoch >= 2


def test_content_column_and_missing_column():
    tok = SimpleTokenizer(vocab_size=500)
    assert _rows(OnlineTokenizedIterableDataset(_docs(20, "content"), tok, seq_len=16), 3) == \
        _rows(OnlineTokenizedIterableDataset(_docs(20, "text"), tok, seq_len=16), 3)
    with pytest.raises(ValueError, match="'text' or 'content'"):
        _rows(OnlineTokenizedIterableDataset([{"body": "x"}], tok, seq_len=4), 1)


def test_rank_shards_are_disjoint():
    tok = SimpleTokenizer(vocab_size=500)
    docs = _docs(64)
    r0 = OnlineTokenizedIterableDataset(docs, tok, seq_len=8, rank=0, world_size=2)
    r1 = OnlineTokenizedIterableDataset(docs, tok, seq_len=8, rank=1, world_size=2)
    assert r0.data == docs[0::2] and r1.data == docs[1::2]


@pytest.mark.parametrize("stateful", [False, True])
def test_streaming_shuffle_is_a_permutation_and_resumes(stateful):
    items = list(range(300))
    make = (lambda: StatefulList(items)) if stateful else (lambda: list(items))
    full = list(shuffle(make(), seed=7, buffer_size=32))
    assert sorted(full) == items and full != items
    for cut in (5, 150, 290):  # while filling / streaming, and inside the final drain
        s = shuffle(make(), seed=7, buffer_size=32)
        it = iter(s)
        head = [next(it) for _ in range(cut)]
        sd = s.state_dict()
        t = shuffle(make(), seed=7, buffer_size=32)
        t.load_state_dict(sd)
        assert head + list(t) == full, cut


def test_shuffled_stream_under_the_tokenizing_dataset_resumes():
    tok = SimpleTokenizer(vocab_size=500)
    mk = lambda: OnlineTokenizedIterableDataset(shuffle(StatefulList(_docs(300)), seed=3, buffer_size=16), tok, seq_len=32,
                                                docs_per_batch=8)
    full = _rows(mk(), 50)
    a = mk()
    it = iter(a)
    head = [next(it)["input_ids"].tolist() for _ in range(11)]
    b = mk()
    b.load_state_dict(a.state_dict())
    assert head + _rows(b, 39) == full


def test_build_dataset_falls_back_to_map_style_when_the_stream_has_too_few_shards():
    calls = []

    class MapStyle:
        def __init__(self):
            self.ops = []

        def shuffle(self, seed):
            self.ops.append(("shuffle", seed))
            return self

        def to_iterable_dataset(self, num_shards):
            self.ops.append(("shards", num_shards))
            return self

    def loader(path, streaming=False, **kw):
        calls.append((path, streaming))
        return StatefulList(_docs(10), num_shards=2) if streaming else MapStyle()

    ds = build_dataset("corpus", streaming=True, dp_degree=2, num_workers=4, seed=1, loader=loader)
    assert calls == [("corpus", True), ("corpus", False)]
    assert isinstance(ds, MapStyle) and ds.ops == [("shuffle", 1), ("shards", 8)]
    calls.clear()
    ds = build_dataset("corpus", streaming=True, dp_degree=1, num_workers=2, seed=1, loader=loader)  # 2 shards suffice
    assert calls == [("corpus", True)] and isinstance(ds, ShuffledExampleStream) and ds.buffer_size == 1024


def test_build_dataset_mixture_checks_and_interleaves():
    loader = lambda path, streaming=False, **kw: StatefulList(_docs(40, "text" if path == "a" else "content"), 8)
    with pytest.raises(ValueError, match="probabilities are required"):
        build_dataset("a,b", streaming=True, loader=loader)
    with pytest.raises(ValueError, match="must match"):
        build_dataset("a,b", data_probs="1.0", streaming=True, loader=loader)
    mix = build_dataset("a,b", data_probs="0.5,0.5", streaming=True, dp_degree=1, num_workers=1, seed=5, loader=loader)
    assert isinstance(mix, InterleavedStreams)
    assert all(m.buffer_size == 512 for m in mix.members)
    out = list(mix)
    assert len(out) >= 80  # all_exhausted: every member was read to its end at least once
    assert {("text" in x) for x in out} == {True, False}


# ---------------------------------------------------------------------------------------------------------------
# collator (flame/data.py:389-496)
# ---------------------------------------------------------------------------------------------------------------
def test_collator_varlen_eos_rule_and_context_split():
    tok = SimpleTokenizer(vocab_size=100, eos_token_id=2)
    row = torch.tensor([5, 6, 2, 7, 8, 9, 10, 2, 11, 12])  # documents end AFTER each EOS; the tail has no EOS
    out = DataCollatorForLanguageModeling(tok, varlen=True)([{"input_ids": row}])
    assert out["cu_seqlens"].tolist() == [0, 3, 8, 10] and out["cu_seqlens"].dtype == torch.int32
    assert out["input_ids"].shape == (1, 10) and torch.equal(out["labels"], out["input_ids"])  # no boundary masking
    out = DataCollatorForLanguageModeling(tok, context_len=2, varlen=True)([{"input_ids": row}])
    assert out["cu_seqlens"].tolist() == [0, 2, 3, 5, 7, 8, 10]
    row_eos_last = torch.tensor([5, 2, 7, 2])
    assert DataCollatorForLanguageModeling(tok, varlen=True)([row_eos_last])["cu_seqlens"].tolist() == [0, 2, 4]


def test_collator_varlen_prefers_bos_over_eos():
    tok = SimpleTokenizer(vocab_size=100, bos_token_id=1, eos_token_id=2)
    row = torch.tensor([1, 5, 2, 1, 7, 8, 2, 1, 9])
    assert DataCollatorForLanguageModeling(tok, varlen=True)([row])["cu_seqlens"].tolist() == [0, 3, 7, 9]
    row_mid = torch.tensor([5, 2, 1, 7, 8])  # the row starts in the middle of a document: a boundary at 0 is added
    assert DataCollatorForLanguageModeling(tok, varlen=True)([row_mid])["cu_seqlens"].tolist() == [0, 2, 5]


def test_collator_varlen_needs_batch_one_and_a_boundary_token():
    tok = SimpleTokenizer(vocab_size=100)
    with pytest.raises(ValueError, match="batch size must be 1"):
        DataCollatorForLanguageModeling(tok, varlen=True)([torch.tensor([1, 2]), torch.tensor([3, 2])])
    with pytest.raises(ValueError, match="BOS or an EOS"):
        DataCollatorForLanguageModeling(SimpleTokenizer(eos_token_id=None), varlen=True)


def test_collator_dense_stacks_and_pads_with_ignore_index():
    tok = SimpleTokenizer(vocab_size=100, pad_token_id=0)
    out = DataCollatorForLanguageModeling(tok)([torch.tensor([5, 6, 7]), torch.tensor([8, 9])])
    assert out["input_ids"].tolist() == [[5, 6, 7], [8, 9, 0]]
    assert out["labels"].tolist() == [[5, 6, 7], [8, 9, -100]]
    assert "cu_seqlens" not in out
    with pytest.raises(ValueError, match="pad token"):
        DataCollatorForLanguageModeling(SimpleTokenizer())([torch.tensor([5, 6, 7]), torch.tensor([8, 9])])


# ---------------------------------------------------------------------------------------------------------------
# loader state (flame/data.py:501-542)
# ---------------------------------------------------------------------------------------------------------------
def test_loader_state_is_keyed_by_rank_and_resumes():
    tok = SimpleTokenizer(vocab_size=500)
    mk = lambda rank: build_dataloader(_docs(300), tok, rank=rank, world_size=2, batch_size=2, seq_len=16)
    a = mk(1)
    it = iter(a)
    head = [next(it)["input_ids"] for _ in range(3)]
    sd = a.state_dict()
    assert list(sd) == ["rank_1"] and isinstance(sd["rank_1"], bytes)
    rest_a = [next(it)["input_ids"] for _ in range(4)]
    b = mk(1)
    b.load_state_dict(sd)
    rest_b = [x["input_ids"] for x in itertools.islice(iter(b), 4)]
    assert all(torch.equal(x, y) for x, y in zip(rest_a, rest_b))
    c = mk(0)
    c.load_state_dict(sd)  # another rank's state is not applied
    first = next(iter(c))["input_ids"]
    assert torch.equal(first, next(iter(mk(0)))["input_ids"])


def test_prefetch_factor_reaches_the_worker_loader():
    tok = SimpleTokenizer(vocab_size=500)
    dl = build_dataloader(_docs(64), tok, rank=0, world_size=1, batch_size=1, seq_len=16, num_workers=1, prefetch_factor=3)
    assert dl._inner is not None and dl._inner.prefetch_factor == 3


def test_offline_tokeniser_columns_and_bits_per_token(tmp_path):
    """``utils/preprocess.py`` writes the reference's columns (flame/utils/preprocess.py:13-122): ``input_ids`` and
    ``bits_per_token`` = 8 * utf-8 bytes / tokens, for ``text`` or ``content`` sources."""
    from flame_b200.utils.preprocess import tokenize

    class Tok:
        def __call__(self, texts):
            return {"input_ids": [[len(w) for w in t.split()] for t in texts]}

    out = tokenize({"text": ["a bb ccc", "héllo wörld"]}, Tok())
    assert out["input_ids"] == [[1, 2, 3], [5, 5]]
    assert out["bits_per_token"][0] == 8.0 * 8 / 3
    assert out["bits_per_token"][1] == 8.0 * len("héllo wörld".encode("utf-8")) / 2
    assert tokenize({"content": ["x y"]}, Tok())["input_ids"] == [[1, 1]]
    datasets = pytest.importorskip("datasets")
    ds = datasets.Dataset.from_dict({"text": ["one two three", "four five"] * 8})
    tok_ds = ds.map(lambda ex: tokenize(ex, Tok()), batched=True, batch_size=4, remove_columns=ds.column_names)
    tok_ds.save_to_disk(str(tmp_path / "tok"))
    back = datasets.load_from_disk(str(tmp_path / "tok"))
    assert back.column_names == ["input_ids", "bits_per_token"] and len(back) == 16 and back[1]["input_ids"] == [4, 4]
