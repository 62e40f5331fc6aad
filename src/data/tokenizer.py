from nanotitan_b200.data.tokenizer import TiktokenTokenizer  # noqa: F401
