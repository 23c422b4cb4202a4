"""Document sources: Nemotron-CC v1 files on Common Crawl's open host (needs network when used).

Same capabilities as the reference (nanonemo/data/sources.py:21-88): list a quality bucket's file
paths, pick files evenly through the crawl history, resumable size-verified downloads with HTTP
Range, a streaming zstd JSON-lines reader, and a round-robin merge so a token budget trims every
file equally. ``requests`` and ``zstandard`` are imported where used, so the module imports offline.
"""

import gzip
import io
import json
import os
from collections.abc import Iterator
from pathlib import Path

CC_BASE = "https://data.commoncrawl.org/"
NEMOTRON_CC_PATHS = CC_BASE + "contrib/Nemotron/Nemotron-CC/data-jsonl.paths.gz"


def nemotron_cc_paths(quality: str = "high", kind: str = "actual") -> list[str]:
    import requests

    r = requests.get(NEMOTRON_CC_PATHS, timeout=60)
    r.raise_for_status()
    needle = f"/quality={quality}/kind={kind}/kind2={kind}/"
    return sorted(p for p in gzip.decompress(r.content).decode().split() if needle in p)


def select_evenly(paths: list[str], n: int) -> list[str]:
    """`n` entries at equal spacing through `paths` (all of them when n >= len)."""
    if n >= len(paths):
        return list(paths)
    return [paths[(i * len(paths)) // n] for i in range(n)]


def download(path: str, raw_dir: Path, chunk_bytes: int = 1 << 22, max_retries: int = 50) -> Path:
    """Fetch CC_BASE + path into raw_dir, continuing a partial file; the final size must match."""
    import requests

    raw_dir = Path(raw_dir)
    dest = raw_dir / Path(path).name
    if dest.exists():
        return dest
    raw_dir.mkdir(parents=True, exist_ok=True)
    part = dest.with_name(dest.name + ".part")
    url = CC_BASE + path
    total = int(requests.head(url, timeout=60).headers["Content-Length"])
    tries = 0
    while (have := part.stat().st_size if part.exists() else 0) < total:
        try:
            with requests.get(url, headers={"Range": f"bytes={have}-"} if have else {}, stream=True, timeout=60) as r:
                r.raise_for_status()
                if have and r.status_code != 206:
                    raise RuntimeError(f"{url}: server ignored the Range request")
                with open(part, "ab") as f:
                    for chunk in r.iter_content(chunk_bytes):
                        f.write(chunk)
        except (requests.ConnectionError, requests.Timeout) as e:
            tries += 1
            if tries > max_retries:
                raise
            print(f"retry {tries} for {dest.name} at byte {part.stat().st_size if part.exists() else 0}: {e}")
    if part.stat().st_size != total:
        raise RuntimeError(f"{dest.name}: {part.stat().st_size} bytes on disk, expected {total}")
    os.replace(part, dest)
    return dest


def iter_jsonl_zstd(path) -> Iterator[dict]:
    import zstandard

    with open(path, "rb") as raw:
        stream = io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(raw), encoding="utf-8")
        for line in stream:
            rec = json.loads(line)
            yield {"id": rec["warc_record_id"], "text": rec["text"]}


def round_robin(iterators: list[Iterator]) -> Iterator:
    """Interleave: one item from each live iterator per round."""
    live = [iter(it) for it in iterators]
    while live:
        nxt = []
        for it in live:
            try:
                yield next(it)
            except StopIteration:
                continue
            nxt.append(it)
        live = nxt
