"""GPT-2 byte-pair tokens through tiktoken, the reference's tokenizer (src/data/tokenizer.py:6-21):
`encode` is `encode_ordinary` (special-token strings in the text are plain text), ids fit in uint16
(vocabulary 50257), which is what the packed token files store."""
from __future__ import annotations

from collections.abc import Iterable


class TiktokenTokenizer:
    def __init__(self, name: str = "gpt2"):
        import tiktoken  # imported here so that the package works where tiktoken is absent

        self._codec = tiktoken.get_encoding(name)

    @property
    def vocab_size(self) -> int:
        return self._codec.n_vocab

    @property
    def eot_token(self) -> int:
        return self._codec.eot_token

    @property
    def enc(self):
        """The underlying tiktoken encoding (the reference exposes it under this name)."""
        return self._codec

    def encode(self, text: str) -> list[int]:
        return self._codec.encode_ordinary(text)

    def encode_documents(self, texts: Iterable[str], append_eot: bool = False) -> list[int]:
        """Concatenated ids of several documents, optionally separated by the end-of-text token."""
        ids: list[int] = []
        for text in texts:
            ids.extend(self._codec.encode_ordinary(text))
            if append_eot:
                ids.append(self.eot_token)
        return ids

    def decode(self, ids: list[int]) -> str:
        return self._codec.decode(list(ids))
