"""GPT-2 BPE through tiktoken (reference: src/data/tokenizer.py:6-21)."""
from __future__ import annotations


class TiktokenTokenizer:
    def __init__(self, name: str = "gpt2"):
        import tiktoken

        self.enc = tiktoken.get_encoding(name)
        self.vocab_size = self.enc.n_vocab
        self.eot_token = self.enc.eot_token

    def encode(self, text: str) -> list[int]:
        return self.enc.encode_ordinary(text)

    def decode(self, ids: list[int]) -> str:
        return self.enc.decode(ids)
