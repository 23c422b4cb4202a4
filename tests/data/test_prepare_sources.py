"""Document pipeline: dedup/filter, per-document split, shard packing, budget, sources helpers, tokenizer laziness."""

import io
import json

import numpy as np
import pytest

from nanonemo_b200.data import prepare as prep
from nanonemo_b200.data import sources, tokenizer
from nanonemo_b200.data.shard import open_shard


def fake_encode_batch(texts):
    return [[ord(c) % 251 for c in t] + [tokenizer.EOT] for t in texts]


def docs(n, length=300):
    return [{"id": f"doc-{i}", "text": (chr(97 + i % 26) * length) + str(i)} for i in range(n)]


def test_dedup_and_filter_counts():
    stats = prep.Stats()
    items = [{"id": "a", "text": "x" * 300}, {"id": "b", "text": "  " + "x" * 300 + " "}, {"id": "c", "text": "short"},
             {"id": "d", "text": "y" * 300}]
    kept = list(prep.dedup_and_filter(items, 200, stats))
    assert [d["id"] for d in kept] == ["a", "d"]
    assert (stats.docs_seen, stats.docs_duplicate, stats.docs_too_short, stats.docs_kept) == (4, 1, 1, 2)


def test_split_is_deterministic_and_roughly_proportional():
    ids = [f"id{i}" for i in range(5000)]
    splits = [prep.assign_split(i, 0.1) for i in ids]
    assert splits == [prep.assign_split(i, 0.1) for i in ids]
    assert 0.07 < splits.count("val") / len(ids) < 0.13
    assert prep.assign_split("x", 0.0) == "train"


def test_prepare_never_splits_a_document_and_writes_manifest(tmp_path):
    m = prep.prepare(docs(60), tmp_path, source={"kind": "test"}, val_frac=0.2, shard_tokens=1000, tokenize_batch_size=7,
                     encode_batch=fake_encode_batch)
    assert m["stats"]["docs_kept"] == 60 and set(m["splits"]) == {"train", "val"}
    total = 0
    for split in m["splits"].values():
        assert len(split["shards"]) >= 1
        for s in split["shards"]:
            toks = np.asarray(open_shard(tmp_path / s["path"]))
            assert toks[-1] == tokenizer.EOT  # a shard always ends at a document boundary
            assert s["n_tokens"] == len(toks)
            total += len(toks)
    assert total == sum(len(t) for t in fake_encode_batch([d["text"] for d in docs(60)]))


def test_prepare_budget_and_empty_split(tmp_path):
    m = prep.prepare(docs(200), tmp_path / "a", source={}, val_frac=0.1, shard_tokens=5000, tokenize_batch_size=5,
                     max_train_tokens=3000, encode_batch=fake_encode_batch)
    assert 3000 <= m["splits"]["train"]["n_tokens"] < 3000 + 5 * 320 * 2
    with pytest.raises(ValueError, match="empty"):
        prep.prepare(docs(1), tmp_path / "b", source={}, val_frac=0.5, encode_batch=fake_encode_batch)


def test_synthetic_dataset_loads(tmp_path):
    from nanonemo_b200.data.loader import TokenLoader

    prep.write_synthetic_dataset(tmp_path, 5000, 600, shard_tokens=2000)
    ld = TokenLoader(tmp_path, "train", 32, 2)
    x, _ = ld.next_batch()
    assert x.shape == (2, 32) and int(x.max()) < 50257
    manifest = json.loads((tmp_path / "manifest.json").read_text())
    assert len(manifest["splits"]["train"]["shards"]) == 3


def test_select_evenly_and_round_robin():
    paths = [f"p{i:03d}" for i in range(100)]
    picked = sources.select_evenly(paths, 4)
    assert picked == ["p000", "p025", "p050", "p075"]
    assert sources.select_evenly(paths[:3], 10) == paths[:3]
    merged = list(sources.round_robin([iter([1, 2, 3]), iter([10]), iter([20, 21])]))
    assert merged == [1, 10, 20, 2, 21, 3]


def test_zstd_jsonl_reader(tmp_path):
    zstandard = pytest.importorskip("zstandard")
    lines = "\n".join(json.dumps({"warc_record_id": f"w{i}", "text": f"t{i}", "extra": 1}) for i in range(5))
    (tmp_path / "f.jsonl.zstd").write_bytes(zstandard.ZstdCompressor().compress(lines.encode()))
    got = list(sources.iter_jsonl_zstd(tmp_path / "f.jsonl.zstd"))
    assert got[0] == {"id": "w0", "text": "t0"} and len(got) == 5


def test_tokenizer_constants_need_no_network():
    assert tokenizer.VOCAB_SIZE == 50257 and tokenizer.EOT == 50256 and tokenizer.TOKENIZER_NAME == "gpt2"


def test_tokenizer_round_trip_if_available():
    try:
        enc = tokenizer.encoder()
    except RuntimeError:
        pytest.skip("GPT-2 vocabulary not cached and no network")
    ids = tokenizer.encode_doc("hello <|endoftext|> world")
    assert ids[-1] == tokenizer.EOT and ids.count(tokenizer.EOT) == 1  # the literal string is not a special token
    assert tokenizer.decode(ids[:-1]) == "hello <|endoftext|> world"
    assert enc.n_vocab == tokenizer.VOCAB_SIZE
