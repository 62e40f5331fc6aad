from nanotitan_b200.data.dataset import PackedTokenDataset, SyntheticTokenDataset  # noqa: F401
