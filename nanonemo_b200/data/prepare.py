"""Raw documents -> token shards + manifest (offline, CPU only).

Stages, each a small pure function over an iterator so they can be tested without I/O
(behaviour as in the reference pipeline, nanonemo/data/prepare.py:41-169): exact de-duplication by
text hash and a minimum-length filter; a train/val split decided per *document id* before
tokenising (a document never straddles the boundary); tokenising in thread-parallel batches;
packing into shards without ever splitting a document across two shards; a manifest with
per-shard sha256 and the filter statistics. ``python -m nanonemo_b200.data.prepare`` is the CLI.
"""

import argparse
import hashlib
import json
from collections.abc import Iterable, Iterator
from dataclasses import asdict, dataclass
from pathlib import Path

import numpy as np

from nanonemo_b200.data import tokenizer
from nanonemo_b200.data.shard import file_sha256, write_shard


@dataclass
class Stats:
    docs_seen: int = 0
    docs_duplicate: int = 0
    docs_too_short: int = 0
    docs_kept: int = 0


def dedup_and_filter(docs: Iterable[dict], min_chars: int, stats: Stats) -> Iterator[dict]:
    seen: set[bytes] = set()
    for doc in docs:
        stats.docs_seen += 1
        text = doc["text"].strip()
        if len(text) < min_chars:
            stats.docs_too_short += 1
        elif (key := hashlib.sha256(text.encode()).digest()) in seen:
            stats.docs_duplicate += 1
        else:
            seen.add(key)
            stats.docs_kept += 1
            yield dict(doc, text=text)


def assign_split(doc_id: str, val_frac: float) -> str:
    """'val' for a fixed pseudo-random `val_frac` of document ids, else 'train'."""
    u = int.from_bytes(hashlib.sha256(doc_id.encode()).digest()[:8], "big") / 2.0**64
    return "val" if u < val_frac else "train"


class ShardWriter:
    """Accumulates whole documents and writes a shard when the next document would overflow it."""

    def __init__(self, out_dir: Path, prefix: str, shard_tokens: int):
        self.out_dir, self.prefix, self.shard_tokens = Path(out_dir), prefix, shard_tokens
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.shards: list[dict] = []
        self.n_tokens = 0
        self._pending: list[np.ndarray] = []
        self._pending_len = 0

    def add(self, tokens) -> None:
        tokens = np.asarray(tokens)
        if self._pending and self._pending_len + len(tokens) > self.shard_tokens:
            self.flush()
        self._pending.append(tokens)
        self._pending_len += len(tokens)
        self.n_tokens += len(tokens)

    def flush(self) -> None:
        if not self._pending:
            return
        name = f"{self.prefix}_{len(self.shards):06d}.bin"
        info = write_shard(self.out_dir / name, np.concatenate(self._pending), tokenizer.TOKENIZER_NAME)
        self.shards.append({"path": name, **info})
        self._pending, self._pending_len = [], 0

    def close(self) -> list[dict]:
        self.flush()
        return self.shards


def prepare(docs: Iterable[dict], out_dir, *, source: dict, min_chars: int = 200, val_frac: float = 0.02,
            shard_tokens: int = 100_000_000, tokenize_batch_size: int = 256, max_train_tokens: int | None = None,
            encode_batch=None) -> dict:
    """Single pass over `docs`; returns the manifest (the caller writes it)."""
    encode_batch = encode_batch or tokenizer.encode_batch
    stats = Stats()
    writers = {s: ShardWriter(out_dir, s, shard_tokens) for s in ("train", "val")}
    texts: dict[str, list[str]] = {"train": [], "val": []}

    def drain(split):
        if texts[split]:
            for ids in encode_batch(texts[split]):
                writers[split].add(ids)
            texts[split] = []

    for doc in dedup_and_filter(docs, min_chars, stats):
        split = assign_split(doc["id"], val_frac)
        texts[split].append(doc["text"])
        if len(texts[split]) >= tokenize_batch_size:
            drain(split)
            if max_train_tokens is not None and writers["train"].n_tokens >= max_train_tokens:
                break  # checked after a drain: overshoots by at most one batch
    for split in texts:
        drain(split)

    splits = {}
    for split, w in writers.items():
        shards = w.close()
        splits[split] = {"n_tokens": sum(s["n_tokens"] for s in shards), "shards": shards}
        if splits[split]["n_tokens"] == 0 and (split == "train" or val_frac > 0):
            raise ValueError(f"{split} split is empty ({stats.docs_kept} docs kept, val_frac={val_frac})")
    return {"tokenizer": tokenizer.TOKENIZER_NAME, "min_chars": min_chars, "val_frac": val_frac,
            "max_train_tokens": max_train_tokens, "source": source, "splits": splits, "stats": asdict(stats)}


def write_synthetic_dataset(out_dir, train_tokens: int, val_tokens: int, seed: int = 0,
                            shard_tokens: int = 1 << 26) -> dict:
    """Uniform-random token shards + manifest in the on-disk format (benchmarks without a corpus)."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    splits = {}
    for split, n in (("train", train_tokens), ("val", val_tokens)):
        shards, left, i = [], n, 0
        while left > 0:
            m = min(left, shard_tokens)
            name = f"{split}_{i:06d}.bin"
            ids = rng.integers(0, tokenizer.VOCAB_SIZE, size=m, dtype=np.uint16)
            shards.append({"path": name, **write_shard(out_dir / name, ids, tokenizer.TOKENIZER_NAME)})
            left, i = left - m, i + 1
        splits[split] = {"n_tokens": n, "shards": shards}
    manifest = {"tokenizer": tokenizer.TOKENIZER_NAME, "source": {"kind": "synthetic_uniform", "seed": seed},
                "splits": splits}
    (out_dir / "manifest.json").write_text(json.dumps(manifest, indent=2))
    return manifest


def load_hf_sample_docs(repo_id: str, path: str) -> Iterator[dict]:
    """One parquet file of a Hugging Face dataset repo (needs network)."""
    import pandas as pd
    from huggingface_hub import hf_hub_download

    frame = pd.read_parquet(hf_hub_download(repo_id, path, repo_type="dataset"))
    for row in frame.itertuples(index=False):
        yield {"id": row.id, "text": row.text}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--source", choices=["hf_sample", "nemotron_cc", "synthetic"], default="hf_sample")
    ap.add_argument("--repo-id", default="nvidia/Nemotron-Pretraining-Dataset-sample")
    ap.add_argument("--hf-path", default="Nemotron-CC-High-Quality/part_000000.parquet")
    ap.add_argument("--cc-quality", default="high")
    ap.add_argument("--cc-files", type=int, default=12)
    ap.add_argument("--raw-dir", type=Path, default=Path("data/raw/nemotron_cc"))
    ap.add_argument("--max-train-tokens", type=int, default=None)
    ap.add_argument("--min-chars", type=int, default=200)
    ap.add_argument("--val-frac", type=float, default=0.02)
    ap.add_argument("--shard-tokens", type=int, default=2_000_000)
    ap.add_argument("--download-only", action="store_true")
    ap.add_argument("--synthetic-train-tokens", type=int, default=1 << 26)
    ap.add_argument("--synthetic-val-tokens", type=int, default=1 << 22)
    a = ap.parse_args(argv)

    if a.source == "synthetic":
        m = write_synthetic_dataset(a.out, a.synthetic_train_tokens, a.synthetic_val_tokens)
        print(json.dumps({k: v["n_tokens"] for k, v in m["splits"].items()}))
        return
    if a.source == "hf_sample":
        docs = load_hf_sample_docs(a.repo_id, a.hf_path)
        source = {"kind": "hf_sample", "repo_id": a.repo_id, "path": a.hf_path}
    else:
        from nanonemo_b200.data import sources

        paths = sources.select_evenly(sources.nemotron_cc_paths(a.cc_quality, "actual"), a.cc_files)
        local = []
        for i, p in enumerate(paths):
            print(f"[{i + 1}/{len(paths)}] {Path(p).name}", flush=True)
            local.append(sources.download(p, a.raw_dir))
        if a.download_only:
            return
        source = {"kind": "nemotron_cc_v1", "quality": a.cc_quality, "kind2": "actual",
                  "files": [{"path": p, "bytes": f.stat().st_size, "sha256": file_sha256(f)}
                            for p, f in zip(paths, local)]}
        docs = sources.round_robin([sources.iter_jsonl_zstd(f) for f in local])
    manifest = prepare(docs, a.out, source=source, min_chars=a.min_chars, val_frac=a.val_frac,
                       shard_tokens=a.shard_tokens, max_train_tokens=a.max_train_tokens)
    (a.out / "manifest.json").write_text(json.dumps(manifest, indent=2))
    print(json.dumps(manifest["stats"]))
    print(json.dumps({k: v["n_tokens"] for k, v in manifest["splits"].items()}))


if __name__ == "__main__":
    main()
