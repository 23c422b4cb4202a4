"""Shard format and loader invariants, on shards of consecutive integers so every token reveals its origin."""

import json

import numpy as np
import pytest

from nanonemo_b200.data.loader import TokenLoader
from nanonemo_b200.data.shard import HEADER_BYTES, ShardError, file_sha256, open_shard, read_header, write_shard


def make_dataset(root, sizes=(1000, 700, 1300), val=400):
    root.mkdir(parents=True, exist_ok=True)
    start, shards = 0, []
    for i, n in enumerate(sizes):
        name = f"train_{i:06d}.bin"
        info = write_shard(root / name, np.arange(start, start + n) % 60000, "gpt2")
        shards.append({"path": name, **info})
        start += n
    vinfo = write_shard(root / "val_000000.bin", np.arange(val), "gpt2")
    manifest = {"tokenizer": "gpt2", "splits": {"train": {"n_tokens": start, "shards": shards},
                                                 "val": {"n_tokens": val, "shards": [{"path": "val_000000.bin", **vinfo}]}}}
    (root / "manifest.json").write_text(json.dumps(manifest))
    return root


def test_shard_round_trip_and_hash(tmp_path):
    toks = np.random.default_rng(0).integers(0, 50257, 5000)
    info = write_shard(tmp_path / "a.bin", toks, "gpt2")
    assert info["n_tokens"] == 5000 and info["sha256"] == file_sha256(tmp_path / "a.bin")
    assert read_header(tmp_path / "a.bin") == {"version": 1, "n_tokens": 5000, "tokenizer": "gpt2"}
    assert np.array_equal(open_shard(tmp_path / "a.bin"), toks)
    assert not (tmp_path / "a.bin.tmp").exists()


def test_shard_rejects_truncated_foreign_and_oversized(tmp_path):
    write_shard(tmp_path / "a.bin", np.arange(100), "gpt2")
    raw = (tmp_path / "a.bin").read_bytes()
    (tmp_path / "cut.bin").write_bytes(raw[:-10])
    with pytest.raises(ShardError, match="truncated"):
        read_header(tmp_path / "cut.bin")
    (tmp_path / "short.bin").write_bytes(raw[:50])
    with pytest.raises(ShardError, match="too short"):
        read_header(tmp_path / "short.bin")
    (tmp_path / "alien.bin").write_bytes(b"X" * HEADER_BYTES)
    with pytest.raises(ShardError, match="magic"):
        read_header(tmp_path / "alien.bin")
    with pytest.raises(ShardError):
        write_shard(tmp_path / "big.bin", np.array([70000]), "gpt2")


def test_targets_are_inputs_shifted_by_one(tmp_path):
    ld = TokenLoader(make_dataset(tmp_path), "train", seq_len=16, micro_batch=4)
    x, y = ld.next_batch()
    assert x.shape == y.shape == (4, 16)
    assert (y[:, :-1] == x[:, 1:]).all() and (y[:, -1] == x[:, -1] + 1).all()


def test_epoch_covers_every_window_once_and_never_crosses_shards(tmp_path):
    T = 16
    ld = TokenLoader(make_dataset(tmp_path), "train", seq_len=T, micro_batch=1)
    n = ld.n_windows
    assert n == (999 // T) + (699 // T) + (1299 // T)
    starts, bounds = [], np.cumsum([0, 1000, 700, 1300])
    for _ in range(n):
        x, y = ld.next_batch()
        first, last = int(x[0, 0]), int(y[0, -1])
        assert last - first == T  # consecutive integers: the window did not jump across a shard
        shard = np.searchsorted(bounds, first, side="right") - 1
        assert last < bounds[shard + 1]
        starts.append(first)
    assert len(set(starts)) == n
    x, _ = ld.next_batch()  # next epoch: another order
    assert ld.micro_step == n + 1


def test_ranks_are_disjoint_and_cover_the_same_stream(tmp_path):
    root = make_dataset(tmp_path)
    single = TokenLoader(root, "train", 16, 4, seed=3)
    r0 = TokenLoader(root, "train", 16, 2, seed=3, rank=0, world_size=2)
    r1 = TokenLoader(root, "train", 16, 2, seed=3, rank=1, world_size=2)
    for _ in range(5):
        a = single.next_batch()[0]
        b = np.concatenate([r0.next_batch()[0].numpy(), r1.next_batch()[0].numpy()])
        assert np.array_equal(a.numpy(), b)


def test_seed_determinism_and_resume_across_epoch(tmp_path):
    root = make_dataset(tmp_path)
    a, b = TokenLoader(root, "train", 16, 4, seed=1), TokenLoader(root, "train", 16, 4, seed=1)
    c = TokenLoader(root, "train", 16, 4, seed=2)
    assert (a.next_batch()[0] == b.next_batch()[0]).all()
    assert not (a.next_batch()[0] == c.next_batch()[0]).all()
    steps = a.n_windows // 4 + 3
    ref = TokenLoader(root, "train", 16, 4, seed=1)
    seq = [ref.next_batch()[0] for _ in range(steps)]
    first = TokenLoader(root, "train", 16, 4, seed=1)
    for _ in range(steps - 4):
        first.next_batch()
    state = first.state_dict()
    resumed = TokenLoader(root, "train", 16, 4, seed=1)
    resumed.load_state_dict(state)
    for i in range(steps - 4, steps):
        assert (resumed.next_batch()[0] == seq[i]).all()
    other = TokenLoader(root, "train", 16, 8, seed=1)
    with pytest.raises(ValueError, match="micro_batch"):
        other.load_state_dict(state)


def test_synthetic_source_is_uniform_and_layout_independent():
    a = TokenLoader("synthetic:200001", "train", 64, 4, seed=0)
    b0 = TokenLoader("synthetic:200001", "train", 64, 2, seed=0, rank=0, world_size=2)
    b1 = TokenLoader("synthetic:200001", "train", 64, 2, seed=0, rank=1, world_size=2)
    xa = a.next_batch()[0]
    assert np.array_equal(xa.numpy(), np.concatenate([b0.next_batch()[0].numpy(), b1.next_batch()[0].numpy()]))
    assert int(xa.max()) < 50257 and int(xa.min()) >= 0
    v = TokenLoader("synthetic:200001", "val", 64, 4, seed=0).next_batch()[0]
    assert not np.array_equal(v.numpy(), xa.numpy())


def test_too_little_data_raises(tmp_path):
    root = make_dataset(tmp_path, sizes=(10,), val=5)
    with pytest.raises(ValueError, match="too little data"):
        TokenLoader(root, "train", 16, 1)
