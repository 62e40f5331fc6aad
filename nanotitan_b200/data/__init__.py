from nanotitan_b200.data.dataset import PackedTokenDataset, SyntheticTokenDataset, write_synthetic_token_file

__all__ = ["PackedTokenDataset", "SyntheticTokenDataset", "write_synthetic_token_file"]
