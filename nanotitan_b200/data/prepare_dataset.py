"""Tokenise TinyStories into the flat uint16 files the trainer reads.

Reference: src/data/prepare_dataset.py:15-35 (HF `roneneldan/TinyStories`, GPT-2
BPE `encode_ordinary`, concatenated, written to data/preprocessed/).  With
``--synthetic N`` no download happens: N uniform-random ids are written instead.
"""
from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np

from nanotitan_b200.data.dataset import write_synthetic_token_file

OUT_DIR = Path("data/preprocessed")


def write_token_file(token_ids, path) -> None:
    """Token ids as the flat little-endian uint16 stream the datasets read (src/data/prepare_dataset.py:9-12)."""
    stream = np.asarray(token_ids, dtype=np.int64)
    if stream.size and (stream.min() < 0 or stream.max() > 65535):
        raise ValueError("token ids do not fit in uint16")
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    stream.astype("<u2").tofile(path)


def tokenize_split(split: str, tokenizer, out_path: Path) -> int:
    from datasets import load_dataset

    ds = load_dataset("roneneldan/TinyStories", split=split)
    chunks = [np.asarray(tokenizer.encode(row["text"]), dtype=np.uint16) for row in ds]
    stream = np.concatenate(chunks) if chunks else np.zeros(0, dtype=np.uint16)
    write_token_file(stream, out_path)
    return int(stream.size)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--synthetic", type=int, default=0, help="write N random tokens per split")
    ap.add_argument("--vocab-size", type=int, default=50257)
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args()
    targets = {"train": OUT_DIR / "tinystories_train.bin", "validation": OUT_DIR / "tinystories_val.bin"}
    if args.synthetic:
        for i, path in enumerate(targets.values()):
            write_synthetic_token_file(path, args.vocab_size, args.synthetic, args.seed + i)
            print(f"wrote {args.synthetic} synthetic tokens to {path}")
        return
    from nanotitan_b200.data.tokenizer import TiktokenTokenizer

    tok = TiktokenTokenizer()
    for split, path in targets.items():
        print(f"{split}: {tokenize_split(split, tok, path)} tokens -> {path}")


if __name__ == "__main__":
    main()
