"""Token datasets.

`PackedTokenDataset` reads the reference's on-disk format: a flat little-endian
uint16 token stream; sample i is the window [i*S, i*S+S+1) split into inputs and
next-token targets (reference: src/data/dataset.py:8-27).  `SyntheticTokenDataset`
produces uniform-random ids of the same shape with no file, for benchmarks.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
from torch.utils.data import Dataset


class PackedTokenDataset(Dataset):
    def __init__(self, path: str | Path, seq_len: int):
        self.path = Path(path)
        self.seq_len = seq_len
        self.tokens = np.memmap(self.path, dtype=np.uint16, mode="r")
        self.num_sequences = (len(self.tokens) - 1) // seq_len  # +1 token for the shifted target

    def __len__(self) -> int:
        return self.num_sequences

    def __getitem__(self, idx: int):
        lo = idx * self.seq_len
        window = torch.from_numpy(self.tokens[lo : lo + self.seq_len + 1].astype(np.int64))
        return window[:-1], window[1:]


class SyntheticTokenDataset(Dataset):
    """Uniform-random ids in [0, vocab); sample i is a pure function of (seed, i)."""

    def __init__(self, vocab_size: int, seq_len: int, num_sequences: int, seed: int = 42):
        self.vocab_size, self.seq_len = vocab_size, seq_len
        self.num_sequences, self.seed = num_sequences, seed

    def __len__(self) -> int:
        return self.num_sequences

    def __getitem__(self, idx: int):
        gen = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        window = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=gen)
        return window[:-1], window[1:]


def write_synthetic_token_file(
    path: str | Path, vocab_size: int, num_tokens: int, seed: int = 42
) -> Path:
    """Write `num_tokens` uniform-random ids as the uint16 stream `PackedTokenDataset` reads."""
    assert vocab_size <= 65536, "uint16 token files hold ids below 65536"
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    rng.integers(0, vocab_size, size=num_tokens, dtype=np.uint16).tofile(path)
    return path
