from glob import glob
from pathlib import Path

import pytest

from nanotitan_b200.config import AppConfig, ModelConfig, load_config, resolve_config_path

CONFIGS = [p for p in glob("configs/*.toml") if not Path(p).name.startswith("sweep_")]


@pytest.mark.parametrize("path", CONFIGS)
def test_checked_in_configs_load(path):
    cfg = load_config(path)
    assert cfg.runtime.num_expert == cfg.model.num_experts


def test_defaults_match_reference_schema():
    cfg = load_config("configs/dist.toml")
    assert cfg.runtime.reducer == "v0" and cfg.runtime.bucket_size == 25
    assert cfg.runtime.ep_size == 1 and cfg.model.moe_router_dtype == "float32"
    assert cfg.optim.lr == pytest.approx(1e-3)  # the string "1e-3" is coerced
    assert cfg.track_backward_time is False


def test_unknown_keys_are_rejected():
    raw = load_config("configs/dist.toml").model_dump(mode="json")
    raw["model"]["not_a_key"] = 1
    with pytest.raises(Exception):
        AppConfig.model_validate(raw)


def test_odd_width_rejected():
    with pytest.raises(Exception):
        ModelConfig(vocab_size=8, d_model=7, d_head=1, n_heads=1, n_layers=1, max_seq_len=4,
                    ffn_in=8, num_experts=1, top_k=1, router_alpha=0.0)


def test_profiler_needs_active_steps():
    raw = load_config("configs/dist.toml").model_dump(mode="json")
    raw["profiler"].update(enabled=True, active_steps=0)
    with pytest.raises(Exception):
        AppConfig.model_validate(raw)


def test_resolve_config_path_falls_back_to_configs_dir():
    assert resolve_config_path("dist.toml") == Path("configs/dist.toml")
    with pytest.raises(FileNotFoundError):
        resolve_config_path("nope.toml")
