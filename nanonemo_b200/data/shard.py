"""Binary token shards, byte-compatible with the reference format (nanonemo/data/shard.py:1-72).

File = 256-byte header + ``n_tokens`` little-endian uint16 ids. Header fields, packed ``<8sIQ32s`` and
zero-padded: magic ``NNMOTOKS``, format version 1, token count, tokenizer name. Writers are atomic
(temp file, fsync, rename); readers verify magic, version and the exact file size before mapping.
"""

import hashlib
import os
import struct
from pathlib import Path

import numpy as np

MAGIC = b"NNMOTOKS"
VERSION = 1
HEADER_BYTES = 256
DTYPE = np.dtype("<u2")
_FMT = struct.Struct("<8sIQ32s")


class ShardError(ValueError):
    pass


def _header(n_tokens: int, tokenizer: str) -> bytes:
    name = tokenizer.encode()
    if len(name) > 32:
        raise ShardError(f"tokenizer name {tokenizer!r} longer than 32 bytes")
    return _FMT.pack(MAGIC, VERSION, n_tokens, name) + b"\0" * (HEADER_BYTES - _FMT.size)


def read_header(path) -> dict:
    path = Path(path)
    size = path.stat().st_size
    with path.open("rb") as f:
        head = f.read(HEADER_BYTES)
    if len(head) != HEADER_BYTES:
        raise ShardError(f"{path}: {size} bytes is too short for a shard header")
    magic, version, n_tokens, name = _FMT.unpack_from(head)
    if magic != MAGIC:
        raise ShardError(f"{path}: bad magic {magic!r}; not a token shard")
    if version != VERSION:
        raise ShardError(f"{path}: shard version {version}, this reader handles {VERSION}")
    want = HEADER_BYTES + n_tokens * DTYPE.itemsize
    if size != want:
        raise ShardError(f"{path}: file is {size} bytes but the header implies {want} (truncated or padded)")
    return {"version": version, "n_tokens": n_tokens, "tokenizer": name.rstrip(b"\0").decode()}


def write_shard(path, tokens, tokenizer: str) -> dict:
    """Atomically write `tokens`; returns {"n_tokens", "sha256"} of the finished file."""
    path = Path(path)
    arr = np.asarray(tokens)
    if arr.size and (arr.min() < 0 or arr.max() > 0xFFFF):
        raise ShardError("token ids do not fit uint16")
    arr = np.ascontiguousarray(arr, dtype=DTYPE)
    head = _header(arr.size, tokenizer)
    digest = hashlib.sha256(head)
    digest.update(arr.tobytes())
    tmp = path.with_name(path.name + ".tmp")
    with tmp.open("wb") as f:
        f.write(head)
        arr.tofile(f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return {"n_tokens": int(arr.size), "sha256": digest.hexdigest()}


def open_shard(path) -> np.memmap:
    """Read-only memory map of a shard's tokens."""
    meta = read_header(path)
    return np.memmap(path, dtype=DTYPE, mode="r", offset=HEADER_BYTES, shape=(meta["n_tokens"],))


def file_sha256(path, chunk_bytes: int = 1 << 24) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(chunk_bytes), b""):
            digest.update(block)
    return digest.hexdigest()
