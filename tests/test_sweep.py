from pathlib import Path

from nanotitan_b200.config import AppConfig, load_config
from nanotitan_b200.sweep import build_runs, dump_toml, launch_command, main


def test_checked_in_sweep_builds_valid_named_runs():
    _, runs = build_runs(Path("configs/sweep_hparams.toml"))
    assert len(runs) == 18
    assert runs[0][0].endswith("optim-lr-0.01__model-dtype-bfloat16")
    assert len({name for name, _ in runs}) == len(runs)
    for name, config in runs:
        assert AppConfig.model_validate(config).run_name == name


def test_generated_toml_round_trips(tmp_path):
    _, runs = build_runs(Path("configs/sweep_hparams.toml"))
    out = tmp_path / "generated.toml"
    out.write_text(dump_toml(runs[0][1]), encoding="utf-8")
    assert load_config(out).run_name == runs[0][0]


def test_launch_world_size_counts_ep():
    _, runs = build_runs(Path("configs/sweep_hparams.toml"))
    cfg = runs[0][1]
    cfg["runtime"].update(dp_size=2, pp_size=2, ep_size=2)
    assert "--nproc-per-node=8" in launch_command(cfg, Path("x.toml"), "INFO")


def test_dry_run_launches_nothing(capsys):
    assert main(["configs/sweep_hparams.toml", "--dry-run"]) == 0
    assert "[18/18]" in capsys.readouterr().out
