"""Import paths of the reference (`src.*`) mapped onto `nanotitan_b200`, so code written against
nanoTitan (`from src.model.model import NanoTitanModel`, `python -m src.train @cfg.toml`) runs unchanged."""
