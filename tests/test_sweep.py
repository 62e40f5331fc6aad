"""The sweep runner: grid expansion over flat config maps, run names, TOML emission, launch sizing."""
import tomllib
from pathlib import Path

import pytest

from nanotitan_b200 import sweep
from nanotitan_b200.config import AppConfig, load_config

SWEEP = Path("configs/sweep_hparams.toml")


@pytest.fixture(scope="module")
def runs():
    return sweep.build_runs(SWEEP)[1]


def test_flat_form_round_trips():
    nested = {"a": 1, "t": {"x": "s", "u": {"deep": [1, 2]}}, "b": False}
    flat = sweep.flatten(nested)
    assert flat == {"a": 1, "t.x": "s", "t.u.deep": [1, 2], "b": False}
    assert sweep.unflatten(flat) == nested


def test_grid_is_the_cartesian_product_in_file_order():
    points = list(sweep.grid_points({"optim.lr": [1, 2, 3], "model.dtype": ["a", "b"]}))
    assert len(points) == 6
    assert points[0] == {"optim.lr": 1, "model.dtype": "a"} and points[1] == {"optim.lr": 1, "model.dtype": "b"}


def test_checked_in_sweep_expands_to_valid_uniquely_named_configs(runs):
    # 6 learning rates x 3 dtypes
    assert len(runs) == 18
    names = [name for name, _ in runs]
    assert len(set(names)) == 18
    assert names[0].endswith("__optim-lr-0.01__model-dtype-bfloat16")
    for name, cfg in runs:
        validated = AppConfig.model_validate(cfg)
        assert validated.run_name == name
        assert validated.runtime.num_expert == validated.model.num_experts


def test_emitted_toml_loads_back_as_the_same_config(tmp_path, runs):
    name, cfg = runs[7]
    text = sweep.dump_toml(cfg)
    assert tomllib.loads(text)["model"]["dtype"] == cfg["model"]["dtype"]
    path = tmp_path / "run.toml"
    path.write_text(text, encoding="utf-8")
    loaded = load_config(path)
    assert loaded.run_name == name
    assert loaded.model_dump(mode="json") == AppConfig.model_validate(cfg).model_dump(mode="json")


def test_unknown_sweep_key_is_rejected(tmp_path):
    bad = tmp_path / "bad.toml"
    bad.write_text(f'base_config = "{Path("configs/dist.toml").resolve()}"\n[parameters]\n"optim.momentum" = [0.9]\n')
    with pytest.raises(KeyError, match="optim.momentum"):
        sweep.build_runs(bad)


def test_launch_uses_one_process_per_rank_of_all_three_dimensions(runs):
    cfg = runs[0][1]
    cfg["runtime"].update(dp_size=2, pp_size=2, ep_size=2)
    cmd = sweep.launch_command(cfg, Path("x.toml"), "INFO")
    assert "--nproc-per-node=8" in cmd and "@x.toml" in cmd and "--log.level=INFO" in cmd


def test_dry_run_prints_every_run_and_starts_none(capsys):
    assert sweep.main([str(SWEEP), "--dry-run"]) == 0
    out = capsys.readouterr().out
    assert "[18/18]" in out and out.count("torch.distributed.run") == 18


def test_reference_entry_path_is_importable():
    import scripts.sweep as entry

    assert entry.build_runs is sweep.build_runs and entry.main is sweep.main


def test_summary_reads_what_the_runs_logged(tmp_path, monkeypatch, capsys):
    import json

    from nanotitan_b200 import sweep

    monkeypatch.chdir(tmp_path)
    runs = [("a", {}), ("b", {}), ("never-started", {})]
    for name, losses in (("a", [5.0, 4.0, 3.0]), ("b", [5.0, 2.0])):
        folder = tmp_path / "runs" / name
        folder.mkdir(parents=True)
        lines = [{"step": i, "train/ce_loss": v, "train/tokens_per_second": 100.0 * (i + 1)} for i, v in enumerate(losses)]
        lines.append({"step": len(losses) - 1, "val/ce_loss": 9.0})  # validation records are not training steps
        (folder / "metrics.jsonl").write_text("\n".join(json.dumps(x) for x in lines) + "\n")
    rows = sweep.summarize(runs, tail=2)
    assert rows[0] == {"run": "a", "steps": 3, "ce_loss": 3.5, "tokens_per_second": 250.0}
    assert rows[1]["ce_loss"] == 3.5 and rows[1]["steps"] == 2
    assert rows[2] == {"run": "never-started", "steps": 0, "ce_loss": None, "tokens_per_second": None}
