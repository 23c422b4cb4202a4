"""Deterministic, resumable, rank-disjoint token-window loader, plus a synthetic token source.

Semantics follow the reference loader (nanonemo/data/loader.py:1-102): each shard is cut into
windows of ``seq_len + 1`` tokens at stride ``seq_len`` (never crossing a shard); epoch ``e`` visits
every window once in the order ``default_rng([seed, e]).permutation``; global sample
``g = (micro_step * world + rank) * B + b`` maps to window ``perm[g // n][g % n]`` so ranks are
disjoint and the whole state is ``micro_step``.

B200-side differences: batches are assembled directly into a ring of pinned int64 staging buffers
(no per-batch ``pin_memory()`` allocation) and copied on a dedicated copy stream so the H2D of the
next micro-batch overlaps compute; ``data_dir="synthetic[:n_tokens]"`` yields uniform-random ids in
[0, 50257) held in memory, for benchmarks and tests on machines without a dataset.
"""

import json
from pathlib import Path

import numpy as np
import torch

from nanonemo_b200.data.shard import open_shard
from nanonemo_b200.data.tokenizer import TOKENIZER_NAME, VOCAB_SIZE


def synthetic_tokens(n_tokens: int, seed: int = 0, vocab: int = VOCAB_SIZE) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=n_tokens, dtype=np.uint16)


class TokenLoader:
    def __init__(self, data_dir, split: str, seq_len: int, micro_batch: int, seed: int = 0, rank: int = 0,
                 world_size: int = 1, device="cpu", pinned_slots: int = 3):
        spec = str(data_dir)
        if spec.startswith("synthetic"):
            n = int(spec.split(":", 1)[1]) if ":" in spec else (1 << 24) + 1  # independent of the layout
            # train and val draw from different streams
            self.shards = [synthetic_tokens(n, seed=seed * 2 + (split != "train") + 1234)]
        else:
            root = Path(data_dir)
            manifest = json.loads((root / "manifest.json").read_text())
            if manifest["tokenizer"] != TOKENIZER_NAME:
                raise ValueError(f"data tokenized with {manifest['tokenizer']!r}, expected {TOKENIZER_NAME!r}")
            self.shards = [open_shard(root / s["path"]) for s in manifest["splits"][split]["shards"]]
        per_shard = np.array([max(0, (len(s) - 1) // seq_len) for s in self.shards], dtype=np.int64)
        self.n_windows = int(per_shard.sum())
        if self.n_windows == 0:
            raise ValueError(f"split {split!r} has no complete window of {seq_len + 1} tokens; too little data")
        self._ends = np.cumsum(per_shard)
        self._starts = self._ends - per_shard
        self.seq_len, self.micro_batch, self.seed = seq_len, micro_batch, seed
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.micro_step = 0
        self._perm_cache: dict[int, np.ndarray] = {}
        self._slots, self._slot = None, 0
        if self.device.type == "cuda":
            self._slots = [torch.empty((micro_batch, seq_len + 1), dtype=torch.int64).pin_memory()
                           for _ in range(pinned_slots)]
            self._events = [None] * pinned_slots
            self._copy_stream = torch.cuda.Stream(device=self.device)
        self.h2d_bytes_per_batch = micro_batch * (seq_len + 1) * 8

    def _permutation(self, epoch: int) -> np.ndarray:
        perm = self._perm_cache.get(epoch)
        if perm is None:
            self._perm_cache = {epoch: np.random.default_rng([self.seed, epoch]).permutation(self.n_windows)}
            perm = self._perm_cache[epoch]
        return perm

    def window_ids(self, micro_step: int) -> np.ndarray:
        """Global window indices of this rank's micro-batch at `micro_step`."""
        g = (micro_step * self.world_size + self.rank) * self.micro_batch + np.arange(self.micro_batch)
        out = np.empty(self.micro_batch, dtype=np.int64)
        for i, (epoch, pos) in enumerate(zip(g // self.n_windows, g % self.n_windows)):
            out[i] = self._permutation(int(epoch))[pos]
        return out

    def _fill(self, dst: np.ndarray, micro_step: int):
        T = self.seq_len
        for b, w in enumerate(self.window_ids(micro_step)):
            s = int(np.searchsorted(self._ends, w, side="right"))
            start = int(w - self._starts[s]) * T
            dst[b] = self.shards[s][start:start + T + 1]

    def next_batch(self):
        """(x, y) int64 of shape (B, T), y shifted by one token; on CUDA the copy is asynchronous."""
        if self._slots is None:
            windows = np.empty((self.micro_batch, self.seq_len + 1), dtype=np.int64)
            self._fill(windows, self.micro_step)
            self.micro_step += 1
            batch = torch.from_numpy(windows)
            return batch[:, :-1], batch[:, 1:]
        i = self._slot
        self._slot = (i + 1) % len(self._slots)
        if self._events[i] is not None:
            self._events[i].synchronize()  # the copy that last used this staging buffer has finished
        self._fill(self._slots[i].numpy(), self.micro_step)
        self.micro_step += 1
        with torch.cuda.stream(self._copy_stream):
            batch = self._slots[i].to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self._events[i] = ev
        torch.cuda.current_stream(self.device).wait_event(ev)
        batch.record_stream(torch.cuda.current_stream(self.device))
        return batch[:, :-1], batch[:, 1:]

    def state_dict(self) -> dict:
        return {"micro_step": self.micro_step, "seed": self.seed, "seq_len": self.seq_len,
                "micro_batch": self.micro_batch, "world_size": self.world_size}

    def load_state_dict(self, state: dict) -> None:
        for key in ("seed", "seq_len", "micro_batch", "world_size"):
            if state[key] != getattr(self, key):
                raise ValueError(f"cannot resume: {key} was {state[key]}, now {getattr(self, key)}")
        self.micro_step = state["micro_step"]


class DeviceBatches:
    """`n` batches of a loader staged on the device once and then served round-robin: a data source
    with no host->device traffic, for device-only timing of the training step."""

    def __init__(self, loader: TokenLoader, n: int):
        self.batches = [tuple(t.clone() for t in loader.next_batch()) for _ in range(n)]
        self.micro_step = 0
        self.loader = loader

    def next_batch(self):
        b = self.batches[self.micro_step % len(self.batches)]
        self.micro_step += 1
        return b
